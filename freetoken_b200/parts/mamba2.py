"""Mamba-2 (state-space duality): a recurrent mixer with a matrix state per head and one decay per head and token.

One projection of the input gives ``[z | x | B | C | dt]`` (``inner = n_heads * v_head_dim`` columns for the gate
``z`` and for ``x``, ``groups * state`` for each of ``B`` and ``C``, one step size per head).  ``x``, ``B`` and ``C``
together pass a short causal convolution over time per channel (with bias) and ``silu``.  Per token and head ``h``
(which reads ``B`` and ``C`` of group ``h // (n_heads / groups)``)::

    dt = softplus(dt + dt_bias)                               no clamp
    S_t = exp(-exp(A_log) dt) S_(t-1) + dt B_t x_t^T          [state, v_head_dim], 32-bit
    y_t = S_t^T C_t + D x_t

``y`` (heads side by side) is multiplied by ``silu(z)``, then RMS-normed in ``norm_groups`` equal parts with one
plain weight over all of it, then projected.  The recurrence is the one of gated linear attention with keys ``B``
times the step size, queries ``C`` and one decay per (token, head): it runs on :func:`ops.gla_scan` (``k_fac``,
``a_head``, ``qk_div`` for the groups), chunked over long portions.  Step sizes, decays, state, the recurrence's
sums, the gate and the norm are 32-bit (:func:`ops.ssm_gates`, :func:`ops.ssm_output`).

Per request the layer keeps the state ``[n_heads, state, v_head_dim]`` and the convolution's last ``taps - 1``
inputs, in one slot of the cache manager's state pool; both start from zero.  The reference has no recurrent mixer.
"""

from __future__ import annotations

from typing import Any, Dict

import torch

from ..config.spec import ParamSpec, PartSpec, StateNeed
from ..errors import ConfigError
from ..kernels import ops
from .base import MIXERS, BuildEnv, Mixer, StepState
from .gla import DEFAULT_CHUNK, chunk_list


@MIXERS.register("mamba2")
class Mamba2(Mixer):
    """params: ``hidden``, ``n_heads``, ``v_head_dim``, ``state``, ``groups``, ``taps``, ``norm_groups``, ``eps`` (of the
    output norm), ``chunk`` (tokens per chunk of a long portion), ``init_std``."""

    graph_safe = False  # running a step twice would advance the state twice
    graph_recordable = True  # everything a step does is decided on the device

    def __init__(self, spec: PartSpec, env: BuildEnv):
        super().__init__(spec, env)
        g = lambda k: int(spec[k])  # noqa: E731
        self.hidden, self.n_heads, self.v_dim, self.state, self.groups = g("hidden"), g("n_heads"), g("v_head_dim"), g("state"), g("groups")
        self.taps = int(spec.get("taps", 4))
        self.norm_groups = int(spec.get("norm_groups", 1))
        self.eps = float(spec.get("eps", 1e-6))
        self.chunk = int(spec.get("chunk", DEFAULT_CHUNK))
        if min(self.hidden, self.n_heads, self.v_dim, self.groups, self.chunk) < 1 or not 1 <= self.state <= 256:
            raise ConfigError("mamba2: heads, head size, groups and chunk must be positive, the state at most 256")
        if self.n_heads % self.groups:
            raise ConfigError("mamba2: n_heads must be a multiple of groups")
        if not 1 <= self.taps <= 16:
            raise ConfigError(f"mamba2: {self.taps} taps (1 to 16 taken)")
        self.inner = self.n_heads * self.v_dim
        if self.norm_groups < 1 or self.inner % self.norm_groups:
            raise ConfigError("mamba2: norm_groups must divide n_heads * v_head_dim")
        self.bc = self.groups * self.state
        self.conv_dim = self.inner + 2 * self.bc
        self.dt_col = self.inner + self.conv_dim
        self.proj_rows = self.dt_col + self.n_heads

    def param_specs(self) -> Dict[str, ParamSpec]:
        std = self.spec.get("init_std")
        std_in, std_out = (float(std[0]), float(std[1])) if std else (0.02, 0.02)
        H = self.n_heads
        f32 = dict(dtype="float32", store="bfloat16")
        return {
            "in_proj.weight": ParamSpec((self.proj_rows, self.hidden), init=("normal", 0.0, std_in)),
            "conv.weight": ParamSpec((self.conv_dim, self.taps), init=("normal", 0.0, 0.4 if std else 0.02), **f32),
            "conv.bias": ParamSpec((self.conv_dim,), init=("normal", 0.0, 0.2 if std else 0.02), **f32),
            "dt_bias": ParamSpec((H,), init=("normal", -1.0 if std else 0.0, 0.5 if std else 0.02), **f32),
            "A_log": ParamSpec((H,), init=("normal", -1.0 if std else 0.0, 0.5 if std else 0.02), **f32),
            "D": ParamSpec((H,), init=("normal", 1.0, 0.2 if std else 0.02), **f32),
            "norm.weight": ParamSpec((self.inner,), init=("normal", 1.0, 0.2 if std else 0.02), **f32),
            "o_proj.weight": ParamSpec((self.hidden, self.inner), init=("normal", 0.0, std_out)),
        }

    def cache_need(self):
        tensors = [("s", (self.n_heads, self.state, self.v_dim), "float32")]
        if self.taps > 1:
            tensors.append(("conv", (self.taps - 1, self.conv_dim), "float32"))
        return StateNeed(tuple(tensors))

    def max_chunks(self, n_tokens: int) -> int:
        return n_tokens // self.chunk + self.env.max_decode_rows + 1

    def workspace_bytes(self, n_tokens: int) -> int:
        item = 4 if self.env.dtype == torch.float32 else 2
        H, N, P = self.n_heads, self.state, self.v_dim
        rows = n_tokens * ((self.proj_rows + self.conv_dim + self.inner + self.hidden) * item + (self.inner + 2 * H) * 4)
        return rows + self.max_chunks(n_tokens) * H * N * (P + 1) * 4

    def prepare(self, builder) -> None:
        """Put the step's chunk lists into its metadata (once per chunk size; the recurrence's other users share them)."""
        name = f"gla.chunks.{self.chunk}"
        found = getattr(builder, "_gla_lists", None)
        if found is None:
            found = builder._gla_lists = {}
        if name not in found:
            chunks, per_seg, single, multi = chunk_list(builder.seg_lens, self.chunk)
            builder.add(name, chunks)
            builder.add(name + ".segments", per_seg)
            found[name] = (chunks.shape[0], single, multi)
        self._step_lists = (name,) + found[name]

    def forward(self, h: torch.Tensor, step: StepState, cache: Any, writes_cache: bool) -> torch.Tensor:
        if not writes_cache:
            raise ConfigError("mamba2: a state cannot be shared between layers")
        T = h.shape[0]
        ws, dt, cap = self.env.workspace, self.env.dtype, self.env.max_step_tokens
        H, N, P, I = self.n_heads, self.state, self.v_dim, self.inner
        f32 = torch.float32
        n_segs = len(step.segments)
        proj = ws.get("mamba2.proj", (T, self.proj_rows), dt, (cap, self.proj_rows))
        ops.linear(h, self.params["in_proj.weight"], proj)
        xbc = ws.get("mamba2.xbc", (T, self.conv_dim), dt, (cap, self.conv_dim))
        ops.conv_act(proj[:, I: self.dt_col], self.params["conv.weight"], self.params["conv.bias"], "silu",
                     cache.tensors["conv"] if self.taps > 1 else None, step.state_slots, step.seg_info, n_segs, xbc)
        step_size = ws.get("mamba2.dt", (T, H), f32, (cap, H))
        dec = ws.get("mamba2.decay_t", (T, H), f32, (cap, H))
        ops.ssm_gates(proj[:, self.dt_col:], self.params["dt_bias"], self.params["A_log"], step_size, dec)
        name, n_chunks, single, multi = self._step_lists
        tensors = step.extras["tensors"]
        carry = decay = None
        if multi:
            most = self.max_chunks(cap)
            carry = ws.get("mamba2.carry", (n_chunks, H, N, P), f32, (most, H, N, P))
            decay = ws.get("mamba2.decay", (n_chunks, H, N), f32, (most, H, N))
        o32 = ws.get("mamba2.o32", (T, H, P), f32, (cap, H, P))
        # queries C, keys B times the step size, values x: where the convolution left them
        ops.gla_scan(xbc[:, I + self.bc:], xbc[:, I: I + self.bc], xbc[:, :I], None, None, 1.0, 1.0, cache.tensors["s"],
                     step.state_slots, step.seg_info, n_segs, tensors[name], n_chunks, tensors[name + ".segments"],
                     single, multi, carry, decay, o32, k_fac=step_size, a_head=dec, qk_div=H // self.groups)
        y = ws.get("mamba2.y", (T, I), dt, (cap, I))
        ops.ssm_output(o32, xbc[:, :I], self.params["D"], proj[:, :I], self.params["norm.weight"], self.norm_groups,
                       self.eps, y)
        out = ws.get("mamba2.out", (T, self.hidden), dt, (cap, self.hidden))
        ops.linear(y, self.params["o_proj.weight"], out)
        return out
