"""Typed Kekopel configuration, read from the design's own config.json keys.

A Kekopel file gives every size and every constant that can differ between models of the design:

* ``vocab``, ``width``, ``norm.eps``, ``canon.taps`` (taps of the short convolution in front of every sub-layer);
* ``layers``: a list, one entry per layer, ``{"type", "mixer": {...}, "mlp": {...} | null}``.
  ``type: "latent_attention"``: ``heads``, ``dim`` (unrotated query/key size per head), ``rot_dim`` (rotated size; the
  key's rotated part is shared by all heads), ``vdim``, ``q_rank`` and ``kv_rank`` (sizes of the latents), ``scale``,
  ``mask.size`` (the sliding window: a token sees itself and the ``size - 1`` before it; no ``mask``: everything),
  ``rot.dims`` and ``rot.base`` (how many leading dimensions of the rotated part turn, neighbours in pairs).
  ``type: "mlstm"``: ``heads``, ``dim``, ``vdim``, ``gate_cap``.
  ``mlp.kind`` is ``"dense"`` (``ff``) or ``"moe"`` (``expert.ff``, ``router.experts``, ``router.top``).

Anything missing or out of range becomes a :class:`ConfigError` naming the key.  The reference has no such
design; the reader follows the shape of its MiniMax-M3 reader (python/freetoken/models/minimax_m3/args.py:78-254).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from ..errors import ConfigError
from .pabavik import _get

ARCHITECTURES = ("Kekopel",)
MAX_POSITION = 1 << 20  # the design has no position limit of its own; tables are sized by the engine's longest sequence


@dataclass(frozen=True)
class KekopelLatentAttention:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    window: Optional[int]
    rot_dims: int
    rot_base: float


@dataclass(frozen=True)
class KekopelMatrixMemory:
    heads: int
    dim: int
    vdim: int
    gate_cap: float


@dataclass(frozen=True)
class KekopelMlp:
    kind: str  # "dense" | "moe"
    ff: int
    experts: int = 0
    top: int = 0


@dataclass(frozen=True)
class KekopelLayer:
    type: str  # "latent_attention" | "mlstm"
    mixer: Any
    mlp: Optional[KekopelMlp]


@dataclass(frozen=True)
class KekopelConfig:
    architecture: str
    vocab: int
    width: int
    norm_eps: float
    taps: int
    layers: Tuple[KekopelLayer, ...]
    torch_dtype: Optional[str] = None

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    @staticmethod
    def from_dict(raw: Mapping[str, Any], num_layers: Optional[int] = None) -> "KekopelConfig":
        arch = raw.get("architecture") or (raw.get("architectures") or [None])[0]
        if arch not in ARCHITECTURES:
            raise ConfigError(f"config.json: architecture {arch!r} is not Kekopel")
        vocab = _get(raw, "vocab", "", int)
        width = _get(raw, "width", "", int)
        if vocab < 1 or width < 1:
            raise ConfigError("config.json: 'vocab' and 'width' must be positive")
        taps = _get(_get(raw, "canon", ""), "taps", "canon.", int)
        if not 1 <= taps <= 16:
            raise ConfigError(f"config.json: 'canon.taps'={taps} must be in [1, 16]")
        raw_layers = _get(raw, "layers", "")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        if num_layers is not None:
            raw_layers = raw_layers[:max(1, num_layers)]
        layers = []
        for i, l in enumerate(raw_layers):
            w = f"layers[{i}]."
            typ = _get(l, "type", w)
            m = _get(l, "mixer", w)
            wm = w + "mixer."
            if typ == "latent_attention":
                mask = m.get("mask")
                rot = m.get("rot") or {}
                rot_dim = _get(m, "rot_dim", wm, int)
                mixer = KekopelLatentAttention(
                    heads=_get(m, "heads", wm, int), dim=_get(m, "dim", wm, int), rot_dim=rot_dim,
                    vdim=_get(m, "vdim", wm, int), q_rank=_get(m, "q_rank", wm, int), kv_rank=_get(m, "kv_rank", wm, int),
                    scale=float(_get(m, "scale", wm, float)),
                    window=None if mask is None else _get(mask, "size", wm + "mask.", int),
                    rot_dims=int(rot.get("dims", rot_dim)), rot_base=float(rot.get("base", 10000.0)))
                if min(mixer.heads, mixer.dim, mixer.vdim, mixer.q_rank, mixer.kv_rank) < 1 or mixer.rot_dim < 0:
                    raise ConfigError(f"config.json: '{wm}heads', 'dim', 'vdim', 'q_rank' and 'kv_rank' must be positive")
                if mixer.window is not None and mixer.window < 1:
                    raise ConfigError(f"config.json: '{wm}mask.size' must be positive")
                if mixer.rot_dims < 0 or mixer.rot_dims % 2 or mixer.rot_dims > mixer.rot_dim:
                    raise ConfigError(f"config.json: '{wm}rot.dims'={mixer.rot_dims} must be even and at most "
                                      f"'rot_dim'={mixer.rot_dim}")
                if mixer.rot_dims and not mixer.rot_base > 0:
                    raise ConfigError(f"config.json: '{wm}rot.base' must be positive")
            elif typ == "mlstm":
                mixer = KekopelMatrixMemory(heads=_get(m, "heads", wm, int), dim=_get(m, "dim", wm, int),
                                            vdim=_get(m, "vdim", wm, int), gate_cap=float(_get(m, "gate_cap", wm, float)))
                if mixer.heads < 1 or mixer.dim < 1 or mixer.vdim < 1 or not mixer.gate_cap > 0:
                    raise ConfigError(f"config.json: '{wm}heads', 'dim', 'vdim' and 'gate_cap' must be positive")
            else:
                raise ConfigError(f"config.json: '{w}type' is {typ!r}; this design's mixers are: 'latent_attention', "
                                  f"'mlstm'")
            mlp = None
            rm = l.get("mlp")
            if rm is not None:
                wf = w + "mlp."
                kind = _get(rm, "kind", wf)
                if kind == "dense":
                    mlp = KekopelMlp("dense", ff=_get(rm, "ff", wf, int))
                elif kind == "moe":
                    ex, ro = _get(rm, "expert", wf), _get(rm, "router", wf)
                    mlp = KekopelMlp("moe", ff=_get(ex, "ff", wf + "expert.", int),
                                     experts=_get(ro, "experts", wf + "router.", int), top=_get(ro, "top", wf + "router.", int))
                    if not 1 <= mlp.top <= mlp.experts:
                        raise ConfigError(f"config.json: '{wf}router.top'={mlp.top} must be in [1, experts={mlp.experts}]")
                else:
                    raise ConfigError(f"config.json: '{wf}kind' is {kind!r}; known: 'dense', 'moe'")
                if mlp.ff < 1:
                    raise ConfigError(f"config.json: '{wf}ff' must be positive")
            layers.append(KekopelLayer(typ, mixer, mlp))
        norm = raw.get("norm") or {}
        return KekopelConfig(architecture=str(arch), vocab=vocab, width=width,
                             norm_eps=float(_get(norm, "eps", "norm.", float)), taps=taps, layers=tuple(layers),
                             torch_dtype=raw.get("torch_dtype"))
