"""Tiny Kekopel configurations for tests; they differ in every size, option and constant.

K1: latent attention and matrix memory side by side, dense and expert feed-forwards, top 2 of 5 experts, windows of 9
    and 20, 3 taps, latents of 24 / 40 (query / key-value), a rotated part of which only some dimensions turn.
K2: one head; a window of 1 (a token sees itself only) and none at all; 2 taps; every expert used by every token
    (3 of 3); a layer without feed-forward; matrix memory with more key channels than values.
K3: nothing is a multiple of 4: width 90, vocabulary 101, heads of 10 / 6, latents of 18 / 22, feed-forwards of 30 / 18;
    5 taps; 8 heads on the one cached row; matrix memory first, so that the stack starts with a recurrent layer.
K5: sharp attention (a large score scale), so that a window one token off or a sink left out moves the logits by
    far more than rounding: windows of 16 (a page's size) and 17, sizes whose cached row is 128 wide.
K4: one tap (no convolution at all), matrix-memory layers only besides one attention layer with 32 heads (more
    than the 32-bit attention tile has rows), top 1.
"""

from __future__ import annotations

ARCH = "Kekopel"
PAGE = 4


def _att(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, window, rot_dims, base):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
         "scale": scale, "rot": {"dims": rot_dims, "base": base}}
    if window is not None:
        m["mask"] = {"size": window}
    return m


def _mem(heads, dim, vdim, cap):
    return {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _moe(ff, experts, top):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def _layer(typ, mixer, mlp):
    return {"type": typ, "mixer": mixer, "mlp": mlp}


def _model(vocab, width, eps, taps, layers):
    return {"architecture": ARCH, "vocab": vocab, "width": width, "norm": {"eps": eps}, "canon": {"taps": taps},
            "layers": layers}


KEKO_1 = _model(200, 64, 1e-5, 3, [
    _layer("latent_attention", _att(4, 16, 8, 12, 24, 40, 0.2, 9, 4, 100.0), _dense(48)),
    _layer("mlstm", _mem(2, 16, 24, 8.0), _moe(32, 5, 2)),
    _layer("latent_attention", _att(2, 8, 16, 20, 16, 24, 0.25, 20, 16, 50.0), _moe(24, 5, 2)),
    _layer("mlstm", _mem(4, 8, 8, 15.0), _dense(40)),
])

KEKO_2 = _model(150, 48, 1e-6, 2, [
    _layer("latent_attention", _att(1, 24, 8, 16, 12, 16, 0.18, 1, 8, 10000.0), _moe(16, 3, 3)),
    _layer("mlstm", _mem(1, 40, 12, 5.0), None),
    _layer("latent_attention", _att(1, 12, 4, 28, 20, 28, 0.3, None, 2, 300.0), _dense(64)),
])

KEKO_3 = _model(101, 90, 1e-5, 5, [
    _layer("mlstm", _mem(3, 10, 14, 12.0), _dense(30)),
    _layer("latent_attention", _att(8, 10, 6, 6, 18, 22, 0.22, 13, 6, 1000.0), _moe(18, 4, 1)),
    _layer("mlstm", _mem(5, 6, 33, 3.0), _moe(18, 7, 3)),
])

KEKO_4 = _model(120, 64, 1e-6, 1, [
    _layer("mlstm", _mem(2, 32, 16, 15.0), _moe(20, 6, 1)),
    _layer("latent_attention", _att(32, 4, 4, 4, 32, 12, 0.4, 300, 4, 500000.0), None),
    _layer("mlstm", _mem(4, 16, 16, 10.0), _dense(32)),
])

KEKO_5 = _model(96, 64, 1e-6, 4, [
    _layer("latent_attention", _att(4, 32, 48, 32, 48, 80, 1.5, 16, 48, 10000.0), _dense(64)),
    _layer("latent_attention", _att(2, 16, 16, 24, 32, 112, 2.0, 17, 16, 10000.0), _moe(32, 4, 2)),
])

ALL = {"K1": KEKO_1, "K2": KEKO_2, "K3": KEKO_3, "K4": KEKO_4, "K5": KEKO_5}
