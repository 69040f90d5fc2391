"""Gated delta rule: a recurrent mixer whose matrix state is corrected towards each token's value.

One projection of the input gives ``[q | k | v | g | b | a]``: queries and keys for ``n_kv_heads`` heads of
``head_dim``, values and an output gate for ``n_heads`` heads of ``v_head_dim`` (head ``h`` reads q/k head
``h // (n_heads / n_kv_heads)``), and two logits per head.  ``q``, ``k`` and ``v`` pass a short causal convolution
over time per channel (no bias) and ``silu``; ``q`` and ``k`` are then made unit vectors per head,
``x / sqrt(sum(x^2) + 1e-6)``, and ``q`` is multiplied by ``head_dim^-1/2``.  Per token and head::

    beta = sigmoid(b)         g = exp(-exp(A_log) softplus(a + dt_bias))
    S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q

so the read-out sees the token's own write.  Each head's ``o`` is divided by its root mean square, multiplied by
one plain weight ``[v_head_dim]`` for all heads and by ``silu`` of the gate, and projected.

Unit norms, ``beta``, ``g``, the state and all of the recurrence's sums are 32-bit (:func:`ops.delta_scan`, which
takes the logits and the convolved rows as they lie and runs a request's tokens in order, the state's columns
spread over threads); the output norm and gate are :func:`ops.gated_heads`.  Per request the layer keeps the state
``S`` (stored column by column, ``[n_heads, v_head_dim, head_dim]``) and the convolution's last ``taps - 1`` inputs in one slot of the cache manager's
state pool; both start from zero.  The reference has no recurrent mixer.
"""

from __future__ import annotations

from typing import Any, Dict

import torch

from ..config.spec import ParamSpec, PartSpec, StateNeed
from ..errors import ConfigError
from ..kernels import ops
from .base import MIXERS, BuildEnv, Mixer, StepState

UNIT_EPS = 1e-6  # inside the root of the unit norms of q and k: fixed by the design


@MIXERS.register("gated_delta")
class GatedDelta(Mixer):
    """params: ``hidden``, ``n_heads``, ``n_kv_heads``, ``head_dim``, ``v_head_dim``, ``taps``, ``eps`` (of the output
    norm), ``init_std``."""

    graph_safe = False  # running a step twice would advance the state twice
    graph_recordable = True  # everything a step does is decided on the device

    def __init__(self, spec: PartSpec, env: BuildEnv):
        super().__init__(spec, env)
        g = lambda k: int(spec[k])  # noqa: E731
        self.hidden, self.n_heads, self.head_dim = g("hidden"), g("n_heads"), g("head_dim")
        self.n_kv_heads = int(spec.get("n_kv_heads") or self.n_heads)
        self.v_dim = int(spec.get("v_head_dim") or self.head_dim)
        self.taps = int(spec.get("taps", 4))
        self.eps = float(spec.get("eps", 1e-6))
        if min(self.hidden, self.n_heads, self.n_kv_heads, self.v_dim) < 1 or not 1 <= self.head_dim <= 256:
            raise ConfigError("gated_delta: heads and head sizes must be positive, keys at most 256")
        if self.n_heads % self.n_kv_heads:
            raise ConfigError("gated_delta: n_heads must be a multiple of n_kv_heads")
        if not 1 <= self.taps <= 16:
            raise ConfigError(f"gated_delta: {self.taps} taps (1 to 16 taken)")
        H, G, D, Dv = self.n_heads, self.n_kv_heads, self.head_dim, self.v_dim
        self.k_col = G * D
        self.v_col = 2 * G * D
        self.conv_dim = self.v_col + H * Dv
        self.g_col = self.conv_dim
        self.b_col = self.g_col + H * Dv
        self.a_col = self.b_col + H
        self.proj_rows = self.a_col + H

    def param_specs(self) -> Dict[str, ParamSpec]:
        std = self.spec.get("init_std")
        std_in, std_out = (float(std[0]), float(std[1])) if std else (0.02, 0.02)
        H, Dv = self.n_heads, self.v_dim
        f32 = dict(dtype="float32", store="bfloat16")
        return {
            "in_proj.weight": ParamSpec((self.proj_rows, self.hidden), init=("normal", 0.0, std_in)),
            "conv.weight": ParamSpec((self.conv_dim, self.taps), init=("normal", 0.0, 0.4 if std else 0.02), **f32),
            "A_log": ParamSpec((H,), init=("normal", -1.0 if std else 0.0, 0.5 if std else 0.02), **f32),
            "dt_bias": ParamSpec((H,), init=("normal", -1.0 if std else 0.0, 0.5 if std else 0.02), **f32),
            "norm.weight": ParamSpec((Dv,), init=("normal", 1.0, 0.2 if std else 0.02), **f32),
            "o_proj.weight": ParamSpec((self.hidden, H * Dv), init=("normal", 0.0, std_out)),
        }

    def cache_need(self):
        tensors = [("s", (self.n_heads, self.v_dim, self.head_dim), "float32")]  # S column by column
        if self.taps > 1:
            tensors.append(("conv", (self.taps - 1, self.conv_dim), "float32"))
        return StateNeed(tuple(tensors))

    def workspace_bytes(self, n_tokens: int) -> int:
        item = 4 if self.env.dtype == torch.float32 else 2
        H, Dv = self.n_heads, self.v_dim
        return n_tokens * ((self.proj_rows + self.conv_dim + H * Dv + self.hidden) * item + H * Dv * 4)

    def forward(self, h: torch.Tensor, step: StepState, cache: Any, writes_cache: bool) -> torch.Tensor:
        if not writes_cache:
            raise ConfigError("gated_delta: a state cannot be shared between layers")
        T = h.shape[0]
        ws, dt, cap = self.env.workspace, self.env.dtype, self.env.max_step_tokens
        H, D, Dv = self.n_heads, self.head_dim, self.v_dim
        n_segs = len(step.segments)
        proj = ws.get("delta.proj", (T, self.proj_rows), dt, (cap, self.proj_rows))
        ops.linear(h, self.params["in_proj.weight"], proj)
        qkv = ws.get("delta.qkv", (T, self.conv_dim), dt, (cap, self.conv_dim))
        ops.conv_act(proj[:, : self.conv_dim], self.params["conv.weight"], None, "silu",
                     cache.tensors["conv"] if self.taps > 1 else None, step.state_slots, step.seg_info, n_segs, qkv)
        o32 = ws.get("delta.o32", (T, H, Dv), torch.float32, (cap, H, Dv))
        ops.delta_scan(qkv[:, : self.k_col], qkv[:, self.k_col: self.v_col], qkv[:, self.v_col:],
                       proj[:, self.b_col: self.a_col], proj[:, self.a_col:], self.params["A_log"], self.params["dt_bias"],
                       D ** -0.5, UNIT_EPS, cache.tensors["s"], step.state_slots, step.seg_info, n_segs, o32)
        o = ws.get("delta.o", (T, H, Dv), dt, (cap, H, Dv))
        ops.gated_heads(o32, proj[:, self.g_col: self.b_col], o, Dv, "silu", self.params["norm.weight"], self.eps)
        out = ws.get("delta.out", (T, self.hidden), dt, (cap, self.hidden))
        ops.linear(o.view(T, H * Dv), self.params["o_proj.weight"], out)
        return out
