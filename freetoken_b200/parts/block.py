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

``hyper_residual``: the residual is carried in ``streams`` copies (hyper-connections), all equal to the embedding at
the start.  Sub-layer ``q`` reads ``u = sum_s in_q[s] x_s``, runs on ``N_q(u)``, and its result ``y`` goes back into
every stream while the streams are mixed, ``x_t <- sum_s mix_q[s, t] x_s + out_q[t] y``; after the last layer the
stream is the sum of the copies.  Without ``streams`` the same code runs one copy with all coefficients 1, which
is the plain pre-norm residual.  With ``token_shift`` the mixer's input is first blended, channel by channel, with
the input it had at the token before: ``h_t + (h_(t-1) - h_t) * shift`` (zeros before a sequence's start); the last
input is per-request state of the block.
"""

from __future__ import annotations

from typing import Any, Dict, Optional

import torch

from ..config.spec import ParamSpec, PartSpec, StateNeed
from ..errors import ConfigError
from ..kernels import ops
from .base import (BLOCKS, FEED_FORWARDS, NORMS, Block, BuildEnv, FeedForward, HyperSum, Mixer, NormedSum, Part, RouteSum, StepState,
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


@BLOCKS.register("hyper_residual")
class HyperResidualBlock(Block):
    """params: ``hidden``, ``streams`` (None or 0: one stream, no coefficients in the file), ``eps`` (of the two RMS
    norms, plain weights), ``token_shift`` (bool), ``last`` (the stack's last layer leaves the streams' sum in the one stream; a layer
    that is handed no pending write of its own streams copies the one stream into every stream first), ``init_std``.

    Tensors: ``norm1``, ``norm2`` ``[hidden]``; with streams ``hc1.in``, ``hc1.out`` ``[S]``, ``hc1.mix`` ``[S, S]``
    (indexed ``[from, to]``) and the same under ``hc2``; ``shift [hidden]``.  A layer without feed-forward has none
    of the second ones."""

    graph_safe = False  # the shift's state moves on with every run of a step
    graph_recordable = True

    def __init__(self, spec: PartSpec, env: BuildEnv, mixer: Mixer, ffn: FeedForward,
                 mixer_name: str, ffn_name: str):
        super().__init__(spec, env, mixer, ffn, mixer_name, ffn_name)
        self.hidden = int(spec["hidden"])
        self.file_streams = int(spec.get("streams") or 0)
        self.streams = max(1, self.file_streams)
        if self.streams > 8:
            raise ConfigError(f"hyper_residual: {self.streams} streams (at most 8 taken)")
        self.eps = float(spec["eps"])
        self.shifts = bool(spec.get("token_shift", False))
        self.last = bool(spec.get("last", False))
        self.has_ffn = not isinstance(ffn, NoFeedForward)
        if not self.shifts:
            self.graph_safe = True
        self._ones = None
        self._shift_w = None

    def children(self) -> Dict[str, Part]:
        out = {self.mixer_name: self.mixer}
        if self.has_ffn:
            out[self.ffn_name] = self.ffn
        return out

    def param_specs(self) -> Dict[str, ParamSpec]:
        wide = self.spec.get("init_std") is not None
        f32 = dict(dtype="float32", store="bfloat16")
        S = self.file_streams
        out: Dict[str, ParamSpec] = {}
        for n in ("1", "2") if self.has_ffn else ("1",):
            out["norm" + n] = ParamSpec((self.hidden,), init=("normal", 1.0, 0.2 if wide else 0.02), **f32)
            if S:
                out[f"hc{n}.in"] = ParamSpec((S,), init=("normal", 1.0 / S, 0.3 / S if wide else 0.02), **f32)
                out[f"hc{n}.out"] = ParamSpec((S,), init=("normal", 1.0, 0.3 if wide else 0.02), **f32)
                out[f"hc{n}.mix"] = ParamSpec((S, S), init=("normal", 1.0 / S, 0.5 / S if wide else 0.02), **f32)
        if self.shifts:
            out["shift"] = ParamSpec((self.hidden,), init=("normal", 0.5 if wide else 0.0, 0.2 if wide else 0.02), **f32)
        return out

    def bind(self, tensors) -> None:
        super().bind(tensors)
        if not self.file_streams:
            dev = self.params["norm1"].device
            self._ones = torch.ones((1, 1), dtype=torch.float32, device=dev)
        if self.shifts:  # h + (h' - h) * shift as a two-tap convolution added to the input: taps (shift, -shift)
            mu = self.params["shift"]
            self._shift_w = torch.stack([mu, -mu], dim=1).contiguous()

    def _hc(self, n: str):
        """(in [S], out [S], mix [S, S]) of sub-layer ``n``."""
        if not self.file_streams:
            return self._ones.view(1), self._ones.view(1), self._ones
        return self.params[f"hc{n}.in"], self.params[f"hc{n}.out"], self.params[f"hc{n}.mix"]

    def state_need(self):
        """The block's own per-request state: the mixer's last input before the shift, 32-bit."""
        if not self.shifts:
            return None
        return StateNeed((("shift", (1, self.hidden), "float32"),))

    def workspace_bytes(self, n_tokens: int) -> int:
        item = 4 if self.env.dtype == torch.float32 else 2
        return n_tokens * self.hidden * (self.streams * 4 + 4 + 2 * item)

    def forward(self, x, residual: torch.Tensor, step: StepState, cache: Any, writes_cache: bool):
        T = residual.shape[0]
        ws, dt, cap = self.env.workspace, self.env.dtype, self.env.max_step_tokens
        S = self.streams
        streams = ws.get("block.streams", (S, cap, self.hidden), torch.float32)[:, :T]
        pending = None
        if isinstance(x, HyperSum) and x.streams.data_ptr() == streams.data_ptr() and x.streams.shape == streams.shape:
            pending = x  # the layer before left its last write to be done with this layer's first read
        elif x is not None:
            x = as_rows(x, None, residual)
            if x is not None:
                StreamSum.of(x).fold(residual)
        init = residual if pending is None else None  # the streams start as copies of the one stream
        in1, out1, mix1 = self._hc("1")
        h = ws.get("block.h", (T, self.hidden), dt, (cap, self.hidden))
        if self.shifts:
            state = step.block_states.get(step.entry)
            if state is None:
                raise ConfigError("hyper_residual: the engine gave the block no state for the token shift")
            h32 = ws.get("block.h_f32", (T, self.hidden), torch.float32, (cap, self.hidden))
            first_out = h32
        else:
            first_out = h
        ops.hyper_step(streams, init_from=init, y=pending.y if pending else None, mix=pending.mix if pending else None,
                       out_w=pending.out if pending else None, in_w=in1, norm_w=self.params["norm1"], eps=self.eps,
                       h_out=first_out)
        if self.shifts:
            ops.short_conv(h32, self._shift_w, state.tensors["shift"], step.state_slots, step.seg_info,
                           len(step.segments), h)
        with nvtx_range(f"mixer {self.mixer.kind}"):
            a = as_rows(self.mixer.forward(h, step, cache, writes_cache))
        if not self.has_ffn:
            if self.last:
                ops.hyper_step(streams, y=a, mix=mix1, out_w=out1, sum_out=residual)
                return None
            return HyperSum(a, streams, mix1, out1)
        in2, out2, mix2 = self._hc("2")
        h2 = ws.get("block.h2", (T, self.hidden), dt, (cap, self.hidden))
        ops.hyper_step(streams, y=a, mix=mix1, out_w=out1, in_w=in2, norm_w=self.params["norm2"], eps=self.eps, h_out=h2)
        with nvtx_range(f"feed-forward {self.ffn.kind}"):
            f = as_rows(self.ffn.forward(h2, step))
        if self.last:
            ops.hyper_step(streams, y=f, mix=mix2, out_w=out2, sum_out=residual)
            return None
        return HyperSum(f, streams, mix2, out2)
