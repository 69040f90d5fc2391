"""Typed Nusudra configuration, read from the design's own config.json keys.

A Nusudra file gives every size and every constant that can differ between models of the design:

* ``vocab``, ``width``, ``norm.eps``, ``embedding.scale`` (the embedding rows are multiplied by it), ``streams`` (how
  many copies of the residual the hyper-connections carry; absent: one plain residual);
* ``layers``: a list, one entry per layer, ``{"type", "mixer": {...}, "mlp": {...} | null}``.
  ``type: "latent_attention"``: ``heads``, ``dim`` (unrotated query/key size per head), ``rot_dim`` (rotated size; the
  key's rotated part is shared by all heads), ``vdim``, ``kv_rank``, ``scale``, ``rot.dims`` and ``rot.base`` (how many
  leading dimensions of the rotated part turn, dimension ``i`` with ``i + dims / 2``).
  ``type: "parallel"``: ``mixer.left`` (softmax attention: ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``) and
  ``mixer.right`` (state space: ``heads``, ``vdim``, ``state``, ``groups``, ``conv`` taps, ``norm_groups``).
  ``type: "delta"``: ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``conv`` taps.
  ``mlp.kind`` is ``"dense"`` (``ff``).

Anything missing or out of range becomes a :class:`ConfigError` naming the key.  The reference has no such
design; the reader follows the shape of its MiniMax-M3 reader (python/freetoken/models/minimax_m3/args.py:78-254).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from ..errors import ConfigError
from .pabavik import _get

ARCHITECTURES = ("Nusudra",)
MAX_POSITION = 1 << 20  # the design has no position limit of its own; tables are sized by the engine's longest sequence


@dataclass(frozen=True)
class NusudraLatentAttention:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    rot_dims: int
    rot_base: float


@dataclass(frozen=True)
class NusudraSinkAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float


@dataclass(frozen=True)
class NusudraStateSpace:
    heads: int
    vdim: int
    state: int
    groups: int
    taps: int
    norm_groups: int


@dataclass(frozen=True)
class NusudraParallel:
    left: NusudraSinkAttention
    right: NusudraStateSpace


@dataclass(frozen=True)
class NusudraDelta:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    taps: int


@dataclass(frozen=True)
class NusudraMlp:
    kind: str  # "dense"
    ff: int


@dataclass(frozen=True)
class NusudraLayer:
    type: str  # "latent_attention" | "parallel" | "delta"
    mixer: Any
    mlp: Optional[NusudraMlp]


def _positive(where: str, **values: int) -> None:
    for k, v in values.items():
        if v < 1:
            raise ConfigError(f"config.json: '{where}{k}'={v} must be positive")


@dataclass(frozen=True)
class NusudraConfig:
    architecture: str
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    streams: Optional[int]
    layers: Tuple[NusudraLayer, ...]
    torch_dtype: Optional[str] = None

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    @staticmethod
    def from_dict(raw: Mapping[str, Any], num_layers: Optional[int] = None) -> "NusudraConfig":
        arch = raw.get("architecture") or (raw.get("architectures") or [None])[0]
        if arch not in ARCHITECTURES:
            raise ConfigError(f"config.json: architecture {arch!r} is not Nusudra")
        vocab = _get(raw, "vocab", "", int)
        width = _get(raw, "width", "", int)
        _positive("", vocab=vocab, width=width)
        streams = raw.get("streams")
        if streams is not None:
            streams = _get(raw, "streams", "", int)
            if not 1 <= streams <= 8:
                raise ConfigError(f"config.json: 'streams'={streams} must be in [1, 8]")
        emb = raw.get("embedding") or {}
        scale = float(_get(emb, "scale", "embedding.", float)) if "scale" in emb else 1.0
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
                rot = m.get("rot") or {}
                rot_dim = _get(m, "rot_dim", wm, int)
                mixer = NusudraLatentAttention(
                    heads=_get(m, "heads", wm, int), dim=_get(m, "dim", wm, int), rot_dim=rot_dim,
                    vdim=_get(m, "vdim", wm, int), kv_rank=_get(m, "kv_rank", wm, int),
                    scale=float(_get(m, "scale", wm, float)), rot_dims=int(rot.get("dims", rot_dim)),
                    rot_base=float(rot.get("base", 10000.0)))
                _positive(wm, heads=mixer.heads, dim=mixer.dim, vdim=mixer.vdim, kv_rank=mixer.kv_rank)
                if mixer.rot_dim < 0 or mixer.rot_dims < 0 or mixer.rot_dims % 2 or mixer.rot_dims > mixer.rot_dim:
                    raise ConfigError(f"config.json: '{wm}rot.dims'={mixer.rot_dims} must be even and at most "
                                      f"'rot_dim'={mixer.rot_dim}")
                if mixer.rot_dims and not mixer.rot_base > 0:
                    raise ConfigError(f"config.json: '{wm}rot.base' must be positive")
            elif typ == "parallel":
                a, b = _get(m, "left", wm), _get(m, "right", wm)
                wl, wr = wm + "left.", wm + "right."
                left = NusudraSinkAttention(heads=_get(a, "heads", wl, int), kv_heads=_get(a, "kv_heads", wl, int),
                                            dim=_get(a, "dim", wl, int), vdim=_get(a, "vdim", wl, int),
                                            scale=float(_get(a, "scale", wl, float)))
                _positive(wl, heads=left.heads, kv_heads=left.kv_heads, dim=left.dim, vdim=left.vdim)
                if left.heads % left.kv_heads:
                    raise ConfigError(f"config.json: '{wl}heads' must be a multiple of 'kv_heads'")
                right = NusudraStateSpace(heads=_get(b, "heads", wr, int), vdim=_get(b, "vdim", wr, int),
                                          state=_get(b, "state", wr, int), groups=_get(b, "groups", wr, int),
                                          taps=_get(b, "conv", wr, int), norm_groups=_get(b, "norm_groups", wr, int))
                _positive(wr, heads=right.heads, vdim=right.vdim, state=right.state, groups=right.groups,
                          conv=right.taps, norm_groups=right.norm_groups)
                if right.heads % right.groups:
                    raise ConfigError(f"config.json: '{wr}heads' must be a multiple of 'groups'")
                if (right.heads * right.vdim) % right.norm_groups:
                    raise ConfigError(f"config.json: '{wr}norm_groups' must divide heads * vdim")
                mixer = NusudraParallel(left, right)
            elif typ == "delta":
                mixer = NusudraDelta(heads=_get(m, "heads", wm, int), kv_heads=_get(m, "kv_heads", wm, int),
                                     dim=_get(m, "dim", wm, int), vdim=_get(m, "vdim", wm, int), taps=_get(m, "conv", wm, int))
                _positive(wm, heads=mixer.heads, kv_heads=mixer.kv_heads, dim=mixer.dim, vdim=mixer.vdim, conv=mixer.taps)
                if mixer.heads % mixer.kv_heads:
                    raise ConfigError(f"config.json: '{wm}heads' must be a multiple of 'kv_heads'")
            else:
                raise ConfigError(f"config.json: '{w}type' is {typ!r}; this design's mixers are: 'latent_attention', "
                                  f"'parallel', 'delta'")
            mlp = None
            rm = l.get("mlp")
            if rm is not None:
                wf = w + "mlp."
                kind = _get(rm, "kind", wf)
                if kind != "dense":
                    raise ConfigError(f"config.json: '{wf}kind' is {kind!r}; known: 'dense'")
                mlp = NusudraMlp("dense", ff=_get(rm, "ff", wf, int))
                _positive(wf, ff=mlp.ff)
            layers.append(NusudraLayer(typ, mixer, mlp))
        norm = raw.get("norm") or {}
        return NusudraConfig(architecture=str(arch), vocab=vocab, width=width,
                             norm_eps=float(_get(norm, "eps", "norm.", float)), embedding_scale=scale, streams=streams,
                             layers=tuple(layers), torch_dtype=raw.get("torch_dtype"))
