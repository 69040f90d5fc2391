"""Arrangements of the parts in one layer.

``prenorm_residual`` (python/freetoken/models/minimax_m3/model.py:53-61): every norm call is
"add the previous sub-layer's output to the residual, then norm the sum":
``r += x; h = N_in(r); a = mixer(h); r += a; h = N_post(r); f = ffn(h)`` and ``f`` travels to
the next layer's first norm.  The residual stream is 32-bit.

``parallel_residual``: one norm feeds both sub-layers, ``r += x; h = N(r); a = mixer(h); f = ffn(h)``,
and ``a + f`` travels to the next layer's norm as a :class:`StreamSum`, so that both are added to
the 32-bit stream in 32 bits, by the kernel that norms.  A layer without feed-forward names the
feed-forward kind ``none``.

``sandwich_residual``: every sub-layer is normed on both sides, ``r += N_1b(mixer(N_1(r)))``, then
``r += N_2b(ffn(N_2(r)))``.  The norm behind a sub-layer, the sum into the 32-bit stream and the norm in
front of the next sub-layer are one kernel: a sub-layer's output travels on as a :class:`NormedSum`.

``conv_postnorm_residual``: the sub-layers read the stream itself through a short causal convolution over time
and are normed on their way out only, ``r += ls1 * g1 * unit(mixer(r + conv1(r)))``, then
``r += ls2 * g2 * unit(ffn(r + conv2(r)))`` (``unit`` divides a row by its root mean square, ``g`` is one number,
``ls`` a vector: together one weight vector of an RMS norm).  With ``depth_mix`` the layer then hands on a learned
mix of the outputs of all layers so far (and the embedding): ``r <- sum_(j <= depth + 1) mix[j] X_j``.  The
convolutions' last inputs are per-request state of the block (:meth:`Block.state_need`).
"""

from __future__ import annotations

from typing import Any, Dict, Optional

import torch

from ..config.spec import ParamSpec, PartSpec, StateNeed
from ..errors import ConfigError
from ..kernels import ops
from .base import (BLOCKS, FEED_FORWARDS, NORMS, Block, BuildEnv, FeedForward, Mixer, NormedSum, Part, RouteSum, StepState,
                   StreamSum, as_rows, nvtx_range)


@BLOCKS.register("prenorm_residual")
class PreNormResidualBlock(Block):
    """params: ``hidden``, ``norm`` (PartSpec used for both norms),
    ``input_norm_name``, ``post_norm_name`` (weight-name parts)."""

    def __init__(self, spec: PartSpec, env: BuildEnv, mixer: Mixer, ffn: FeedForward,
                 mixer_name: str, ffn_name: str):
        super().__init__(spec, env, mixer, ffn, mixer_name, ffn_name)
        self.hidden = int(spec["hidden"])
        self.input_norm = NORMS.build(spec["norm"], env)
        self.post_norm = NORMS.build(spec["norm"], env)
        self.input_norm_name = spec.get("input_norm_name", "input_layernorm")
        self.post_norm_name = spec.get("post_norm_name", "post_attention_layernorm")

    def children(self) -> Dict[str, Part]:
        return {self.input_norm_name: self.input_norm, self.mixer_name: self.mixer,
                self.post_norm_name: self.post_norm, self.ffn_name: self.ffn}

    def workspace_bytes(self, n_tokens: int) -> int:
        item = 4 if self.env.dtype == torch.float32 else 2
        return n_tokens * self.hidden * (2 * item + 4)

    def forward(self, x: Optional[torch.Tensor], residual: torch.Tensor, step: StepState,
                cache: Any, writes_cache: bool) -> torch.Tensor:
        T = residual.shape[0]
        ws, dt, cap = self.env.workspace, self.env.dtype, self.env.max_step_tokens
        h = ws.get("block.h", (T, self.hidden), dt, (cap, self.hidden))
        self.input_norm.add_forward(as_rows(x, self.input_norm, residual), residual, h)
        with nvtx_range(f"mixer {self.mixer.kind}"):
            a = self.mixer.forward(h, step, cache, writes_cache)
        h2 = ws.get("block.h2", (T, self.hidden), dt, (cap, self.hidden))
        h32 = None
        if self.ffn.f32_input_needed(T) and dt != torch.float32:
            h32 = ws.get("block.h2_f32", (T, self.hidden), torch.float32, (cap, self.hidden))
        self.post_norm.add_forward(a, residual, h2, out_f32=h32)
        lazy = getattr(self.ffn, "forward_lazy", None)
        with nvtx_range(f"feed-forward {self.ffn.kind}"):
            return lazy(h2, step, h_f32=h32) if lazy is not None else self.ffn.forward(h2, step, h_f32=h32)


@FEED_FORWARDS.register("none")
class NoFeedForward(FeedForward):
    """A layer without feed-forward: owns nothing, adds nothing."""

    def forward(self, h: torch.Tensor, step: StepState, h_f32: Optional[torch.Tensor] = None):
        return None


@BLOCKS.register("parallel_residual")
class ParallelResidualBlock(Block):
    """params: ``hidden``, ``norm`` (PartSpec of the layer's one norm), ``norm_name`` (weight-name part)."""

    def __init__(self, spec: PartSpec, env: BuildEnv, mixer: Mixer, ffn: FeedForward,
                 mixer_name: str, ffn_name: str):
        super().__init__(spec, env, mixer, ffn, mixer_name, ffn_name)
        self.hidden = int(spec["hidden"])
        self.norm = NORMS.build(spec["norm"], env)
        self.norm_name = spec.get("norm_name", "input_layernorm")
        self.has_ffn = not isinstance(ffn, NoFeedForward)

    def children(self) -> Dict[str, Part]:
        out = {self.norm_name: self.norm, self.mixer_name: self.mixer}
        if self.has_ffn:
            out[self.ffn_name] = self.ffn
        return out

    def workspace_bytes(self, n_tokens: int) -> int:
        item = 4 if self.env.dtype == torch.float32 else 2
        return n_tokens * self.hidden * item

    def forward(self, x, residual: torch.Tensor, step: StepState, cache: Any, writes_cache: bool):
        T = residual.shape[0]
        ws, dt, cap = self.env.workspace, self.env.dtype, self.env.max_step_tokens
        h = ws.get("block.h", (T, self.hidden), dt, (cap, self.hidden))
        self.norm.add_forward(as_rows(x, self.norm, residual), residual, h)
        with nvtx_range(f"mixer {self.mixer.kind}"):
            out = StreamSum().add(self.mixer.forward(h, step, cache, writes_cache))
        if self.has_ffn:
            lazy = getattr(self.ffn, "forward_lazy", None)
            with nvtx_range(f"feed-forward {self.ffn.kind}"):
                out.add(lazy(h, step, h_f32=None) if lazy is not None else self.ffn.forward(h, step))
        return out


@BLOCKS.register("sandwich_residual")
class SandwichResidualBlock(Block):
    """params: ``hidden``, ``norm`` (PartSpec used for all four norms; an RMS norm), ``norm_names`` (weight-name
    parts of the norms in front of and behind the mixer, in front of and behind the feed-forward)."""

    def __init__(self, spec: PartSpec, env: BuildEnv, mixer: Mixer, ffn: FeedForward,
                 mixer_name: str, ffn_name: str):
        super().__init__(spec, env, mixer, ffn, mixer_name, ffn_name)
        self.hidden = int(spec["hidden"])
        self.has_ffn = not isinstance(ffn, NoFeedForward)
        self.names = tuple(spec.get("norm_names", ("norm1", "norm1b", "norm2", "norm2b")))
        self.mixer_in = NORMS.build(spec["norm"], env)
        self.mixer_out = NORMS.build(spec["norm"], env)
        self.ffn_in = NORMS.build(spec["norm"], env) if self.has_ffn else None
        self.ffn_out = NORMS.build(spec["norm"], env) if self.has_ffn else None
        for n in (self.mixer_in, self.mixer_out):
            if not getattr(n, "takes_normed_sum", False):
                raise ConfigError("sandwich_residual: its norms are RMS norms (they take a NormedSum)")

    def children(self) -> Dict[str, Part]:
        out = {self.names[0]: self.mixer_in, self.mixer_name: self.mixer, self.names[1]: self.mixer_out}
        if self.has_ffn:
            out.update({self.names[2]: self.ffn_in, self.ffn_name: self.ffn, self.names[3]: self.ffn_out})
        return out

    def workspace_bytes(self, n_tokens: int) -> int:
        item = 4 if self.env.dtype == torch.float32 else 2
        return n_tokens * self.hidden * (2 * item + 4)

    def forward(self, x, residual: torch.Tensor, step: StepState, cache: Any, writes_cache: bool):
        T = residual.shape[0]
        ws, dt, cap = self.env.workspace, self.env.dtype, self.env.max_step_tokens
        h = ws.get("block.h", (T, self.hidden), dt, (cap, self.hidden))
        self.mixer_in.add_forward(as_rows(x, self.mixer_in, residual), residual, h)
        with nvtx_range(f"mixer {self.mixer.kind}"):
            a = NormedSum(self.mixer.forward(h, step, cache, writes_cache), self.mixer_out)
        if not self.has_ffn:
            return a
        h2 = ws.get("block.h2", (T, self.hidden), dt, (cap, self.hidden))
        h32 = None
        if self.ffn.f32_input_needed(T) and dt != torch.float32:
            h32 = ws.get("block.h2_f32", (T, self.hidden), torch.float32, (cap, self.hidden))
        self.ffn_in.add_forward(a, residual, h2, out_f32=h32)
        lazy = getattr(self.ffn, "forward_lazy", None)
        with nvtx_range(f"feed-forward {self.ffn.kind}"):
            f = lazy(h2, step, h_f32=h32) if lazy is not None else self.ffn.forward(h2, step, h_f32=h32)
        return NormedSum(f, self.ffn_out)


@BLOCKS.register("conv_postnorm_residual")
class ConvPostNormResidualBlock(Block):
    """params: ``hidden``, ``taps`` (of the convolutions; 1 = none), ``eps`` (of the output norms), ``depth`` (the
    layer's place in the stack, from 0), ``n_layers``, ``depth_mix`` (bool), ``init_std``.

    Tensors: ``norm1``, ``norm2`` (one number each), ``ls1``, ``ls2`` ``[hidden]``, ``canon1``, ``canon2``
    ``[hidden, taps]``, ``dwa [depth + 2]``; a layer without feed-forward has none of the second ones."""

    graph_safe = False  # the convolutions' state moves on with every run of a step
    graph_recordable = True

    def __init__(self, spec: PartSpec, env: BuildEnv, mixer: Mixer, ffn: FeedForward,
                 mixer_name: str, ffn_name: str):
        super().__init__(spec, env, mixer, ffn, mixer_name, ffn_name)
        self.hidden = int(spec["hidden"])
        self.taps = int(spec.get("taps", 1))
        self.eps = float(spec["eps"])
        self.depth = int(spec.get("depth", 0))
        self.n_layers = int(spec.get("n_layers", self.depth + 1))
        self.mixes = bool(spec.get("depth_mix", False))
        self.has_ffn = not isinstance(ffn, NoFeedForward)
        if not 1 <= self.taps <= 16:
            raise ConfigError(f"conv_postnorm_residual: {self.taps} taps (1 to 16 taken)")
        if not 0 <= self.depth < self.n_layers:
            raise ConfigError("conv_postnorm_residual: depth must lie within the stack")
        self._w1 = self._w2 = None

    def children(self) -> Dict[str, Part]:
        out = {self.mixer_name: self.mixer}
        if self.has_ffn:
            out[self.ffn_name] = self.ffn
        return out

    def param_specs(self) -> Dict[str, ParamSpec]:
        wide = self.spec.get("init_std") is not None
        f32 = dict(dtype="float32", store="bfloat16")
        out: Dict[str, ParamSpec] = {}
        for n in ("1", "2") if self.has_ffn else ("1",):
            out["norm" + n] = ParamSpec((), init=("normal", 1.0, 0.1 if wide else 0.02), **f32)
            out["ls" + n] = ParamSpec((self.hidden,), init=("normal", 0.5 if wide else 1.0, 0.1 if wide else 0.02), **f32)
            out["canon" + n] = ParamSpec((self.hidden, self.taps), init=("normal", 0.0, 0.3 if wide else 0.02), **f32)
        if self.mixes:
            out["dwa"] = ParamSpec((self.depth + 2,), init=("normal", 1.0 / (self.depth + 2), 0.2 if wide else 0.02), **f32)
        return out

    def bind(self, tensors) -> None:
        super().bind(tensors)
        self._w1 = (self.params["norm1"] * self.params["ls1"]).contiguous()
        self._w2 = (self.params["norm2"] * self.params["ls2"]).contiguous() if self.has_ffn else None

    def state_need(self):
        """The block's own per-request state: each convolution's last ``taps - 1`` inputs, 32-bit."""
        if self.taps == 1:
            return None
        names = ("conv1", "conv2") if self.has_ffn else ("conv1",)
        return StateNeed(tuple((n, (self.taps - 1, self.hidden), "float32") for n in names))

    def workspace_bytes(self, n_tokens: int) -> int:
        item = 4 if self.env.dtype == torch.float32 else 2
        hist = (self.n_layers + 1) * n_tokens * self.hidden * 4 if self.mixes else 0
        return n_tokens * self.hidden * 2 * item + hist

    def _add_normed(self, y, weight: torch.Tensor, residual: torch.Tensor) -> None:
        """``residual += unit(y) * weight`` (``y`` rows, or an expert layer's routes still to be summed)."""
        if isinstance(y, RouteSum):
            ops.postnorm_add_norm(y.y, (y.pos, y.top_k, y.shared), weight, self.eps, False, residual)
        else:
            ops.postnorm_add_norm(y, None, weight, self.eps, False, residual)

    def forward(self, x, residual: torch.Tensor, step: StepState, cache: Any, writes_cache: bool):
        if isinstance(x, NormedSum):  # (whatever a block of another kind left to be added)
            x.fold(residual)
        elif x is not None:
            StreamSum.of(x).fold(residual)
        T = residual.shape[0]
        ws, dt, cap = self.env.workspace, self.env.dtype, self.env.max_step_tokens
        state = step.block_states.get(step.entry) if self.taps > 1 else None
        if self.taps > 1 and state is None:
            raise ConfigError("conv_postnorm_residual: the engine gave the block no state")
        n_segs = len(step.segments)
        hist = None
        if self.mixes:
            hist = ws.get("block.history", (self.n_layers + 1, cap, self.hidden), torch.float32)
            if self.depth == 0:
                hist[0, :T].copy_(residual)
        h = ws.get("block.h", (T, self.hidden), dt, (cap, self.hidden))
        ops.short_conv(residual, self.params["canon1"], state.tensors["conv1"] if state else None, step.state_slots,
                       step.seg_info, n_segs, h)
        with nvtx_range(f"mixer {self.mixer.kind}"):
            a = self.mixer.forward(h, step, cache, writes_cache)
        self._add_normed(a, self._w1, residual)
        if self.has_ffn:
            h2 = ws.get("block.h2", (T, self.hidden), dt, (cap, self.hidden))
            ops.short_conv(residual, self.params["canon2"], state.tensors["conv2"] if state else None, step.state_slots,
                           step.seg_info, n_segs, h2)
            lazy = getattr(self.ffn, "forward_lazy", None)
            with nvtx_range(f"feed-forward {self.ffn.kind}"):
                f = lazy(h2, step, h_f32=None) if lazy is not None else self.ffn.forward(h2, step)
            self._add_normed(f, self._w2, residual)
        if self.mixes:
            ops.depth_mix(hist, self.depth + 1, self.params["dwa"], residual[:T])
        return None
