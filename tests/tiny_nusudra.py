"""Tiny Nusudra configurations for tests; they differ in every size, option and constant.

N1: the three mixers in the order delta rule, pair, latent attention; two streams; fewer key heads than heads in the
    delta rule and in the pair's attention, whose values are wider than its keys; two groups in the state-space layer;
    taps of 3 and 2; a layer without feed-forward.
N2: no streams at all (the plain residual); nothing is a multiple of 4: width 90, vocabulary 101; one head everywhere;
    one tap (no convolution state) in the delta rule, five in the state-space layer; one norm group; as many key heads
    as heads.
N3: four streams, latent attention first; sharp attention (large score scales), so that a sink or a distance bias left
    out, or a key one place off, moves the logits by far more than rounding; a cached latent row of 128 (the
    tensor-core attention kernel's size); key channels beyond 32 and value columns beyond 32 in the delta rule.
N4: one stream with coefficients of its own; a state of 24 and heads of 40 (no powers of two); six heads on three
    key heads in the pair's attention; three norm groups; the pair first; a feed-forward narrower than the model.
"""

from __future__ import annotations

ARCH = "Nusudra"
PAGE = 4


def _latent(heads, dim, rot_dim, vdim, kv_rank, scale, base):
    return {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale,
            "rot": {"dims": rot_dim, "base": base}}


def _pair(left, right):
    return {"left": left, "right": right}


def _att(heads, kv_heads, dim, vdim, scale):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}


def _ssm(heads, vdim, state, groups, conv, norm_groups):
    return {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups}


def _delta(heads, kv_heads, dim, vdim, conv):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}


def _layer(typ, mixer, ff):
    return {"type": typ, "mixer": mixer, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def _model(vocab, width, eps, scale, streams, layers):
    raw = {"architecture": ARCH, "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": scale},
           "layers": layers}
    if streams is not None:
        raw["streams"] = streams
    return raw


NUSU_1 = _model(200, 64, 1e-5, 2.0, 2, [
    _layer("delta", _delta(4, 2, 16, 24, 3), 48),
    _layer("parallel", _pair(_att(4, 2, 16, 24, 0.3), _ssm(4, 8, 16, 2, 2, 4)), None),
    _layer("latent_attention", _latent(3, 8, 8, 12, 20, 0.25, 100.0), 40),
    _layer("delta", _delta(2, 2, 8, 8, 4), 56),
])

NUSU_2 = _model(101, 90, 1e-6, 1.0, None, [
    _layer("parallel", _pair(_att(1, 1, 10, 10, 0.35), _ssm(1, 30, 6, 1, 5, 1)), 30),
    _layer("delta", _delta(1, 1, 22, 14, 1), None),
    _layer("latent_attention", _latent(1, 12, 4, 28, 26, 0.3, 300.0), 64),
])

NUSU_3 = _model(160, 96, 1e-5, 1.5, 4, [
    _layer("latent_attention", _latent(6, 16, 32, 16, 96, 1.2, 10000.0), 64),
    _layer("parallel", _pair(_att(2, 2, 32, 32, 1.5), _ssm(3, 16, 8, 1, 4, 1)), 80),
    _layer("delta", _delta(2, 1, 48, 40, 2), 72),
])

NUSU_4 = _model(120, 72, 1e-5, 0.7, 1, [
    _layer("parallel", _pair(_att(6, 3, 8, 12, 0.4), _ssm(6, 6, 24, 3, 3, 3)), 36),
    _layer("delta", _delta(3, 1, 40, 10, 4), 24),
    _layer("latent_attention", _latent(2, 24, 6, 10, 30, 0.2, 50.0), None),
    _layer("parallel", _pair(_att(2, 1, 16, 16, 0.25), _ssm(2, 18, 12, 2, 4, 2)), 48),
])

ALL = {"N1": NUSU_1, "N2": NUSU_2, "N3": NUSU_3, "N4": NUSU_4}
