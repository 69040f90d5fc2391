"""Matrix memory with exponential gates (the mLSTM layer of xLSTM): a recurrent mixer.

Per token and head, with ``q, k`` of size ``D`` (``q`` scaled by ``D^-1/2``), ``v`` of size ``Dv``, a log input
gate ``i_t = cap tanh((W_i h_t + b_i) / cap)`` and a log forget gate ``f_t = logsigmoid(cap tanh((W_f h_t + b_f) / cap))``::

    m_t = max(f_t + m_(t-1), i_t)                                         m_0 = 0
    S_t = e^(f_t + m_(t-1) - m_t) S_(t-1) + e^(i_t - m_t) k_t v_t^T       n_t likewise with k_t alone
    o_t = S_t^T q_t / (max(|n_t . q_t|, e^(-m_t)) + 1e-6)

Each head's ``o_t`` is divided by its root mean square, multiplied by a weight (one per channel of all heads) and
by ``sigmoid(W_g h_t)``, and projected.

The state is ``S_t``, ``n_t`` (one tensor ``[H, D, Dv + 1]``: ``n`` is the recurrence of one more value column
that is 1 for every token) and ``m_t``.  With ``m`` known, the recurrence is linear, with one decay ``e^(f_t + m_(t-1)
- m_t)`` per head and token and keys times ``e^(i_t - m_t)`` (both at most 1, whatever the gates' cap):
:func:`ops.mlstm_gates` scans ``m`` and writes both factors, and :func:`ops.gla_scan` runs the recurrence, chunked over
long portions: it reads ``q, k, v`` where the projection left them, multiplies a token's keys by their factor in 32
bits as it stages them and adds the column of ones itself.  Gates, state, the recurrence's sums and the output's norm
are 32-bit;
the projections are library products.  The state lives in a slot of the cache manager's state pool and starts
from zero (and ``m`` from 0) for a request's first tokens.  The reference has no recurrent mixer.
"""

from __future__ import annotations

from typing import Any, Dict

import torch

from ..config.spec import ParamSpec, PartSpec, StateNeed
from ..errors import ConfigError
from ..kernels import ops
from .base import MIXERS, BuildEnv, Mixer, StepState
from .gla import DEFAULT_CHUNK, chunk_list


@MIXERS.register("mlstm")
class MatrixMemory(Mixer):
    """params: ``hidden``, ``n_heads``, ``head_dim`` (keys and queries), ``v_head_dim``, ``gate_cap``, ``eps`` (of the
    output's unit norm), ``chunk`` (tokens per chunk of a long portion), ``init_std``."""

    graph_safe = False  # running a step twice would advance the state twice
    graph_recordable = True  # everything a step does is decided on the device

    def __init__(self, spec: PartSpec, env: BuildEnv):
        super().__init__(spec, env)
        self.hidden = int(spec["hidden"])
        self.n_heads = int(spec["n_heads"])
        self.head_dim = int(spec["head_dim"])
        self.v_dim = int(spec.get("v_head_dim") or self.head_dim)
        self.cap = float(spec["gate_cap"])
        self.eps = float(spec.get("eps", 1e-6))
        self.chunk = int(spec.get("chunk", DEFAULT_CHUNK))
        if self.n_heads < 1 or not 1 <= self.head_dim <= 256 or self.v_dim < 1 or self.chunk < 1:
            raise ConfigError("mlstm: heads, head sizes (keys at most 256) and chunk must be positive")
        if not self.cap > 0:
            raise ConfigError("mlstm: gate_cap must be positive")
        H, D, Dv = self.n_heads, self.head_dim, self.v_dim
        self.g_row = H * (2 * D + Dv)
        self.proj_rows = self.g_row + H * Dv

    def param_specs(self) -> Dict[str, ParamSpec]:
        std = self.spec.get("init_std")
        std_in, std_out = (float(std[0]), float(std[1])) if std else (0.02, 0.02)
        H, Dv = self.n_heads, self.v_dim
        return {
            "in_proj.weight": ParamSpec((self.proj_rows, self.hidden), init=("normal", 0.0, std_in)),  # q, k, v, gate
            "gate_proj.weight": ParamSpec((2 * H, self.hidden), init=("normal", 0.0, std_in)),       # i, f
            "gate_proj.bias": ParamSpec((2 * H,), "float32", ("normal", 1.0 if std else 0.0, 1.0 if std else 0.02),
                                        store="bfloat16"),
            "norm.weight": ParamSpec((H * Dv,), "float32", ("normal", 1.0, 0.2 if std else 0.02), store="bfloat16"),
            "o_proj.weight": ParamSpec((self.hidden, H * Dv), init=("normal", 0.0, std_out)),
        }

    def cache_need(self):
        H, D, Dv = self.n_heads, self.head_dim, self.v_dim
        return StateNeed((("s", (H, D, Dv + 1), "float32"), ("m", (H,), "float32")))

    def max_chunks(self, n_tokens: int) -> int:
        return n_tokens // self.chunk + self.env.max_decode_rows + 1

    def workspace_bytes(self, n_tokens: int) -> int:
        item = 4 if self.env.dtype == torch.float32 else 2
        H, D, Dv = self.n_heads, self.head_dim, self.v_dim
        rows = n_tokens * ((self.proj_rows + H * Dv + self.hidden) * item + (H * (Dv + 1) + 5 * H) * 4)
        return rows + self.max_chunks(n_tokens) * H * D * (Dv + 2) * 4

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
            raise ConfigError("mlstm: a state cannot be shared between layers")
        T = h.shape[0]
        ws, dt, cap = self.env.workspace, self.env.dtype, self.env.max_step_tokens
        H, D, Dv = self.n_heads, self.head_dim, self.v_dim
        f32 = torch.float32
        proj = ws.get("mlstm.proj", (T, self.proj_rows), dt, (cap, self.proj_rows))
        ops.linear(h, self.params["in_proj.weight"], proj)
        pre = ws.get("mlstm.pre", (T, 2 * H), f32, (cap, 2 * H))
        ops.linear_f32(h, self.params["gate_proj.weight"], pre)
        kf = ws.get("mlstm.key_fac", (T, H), f32, (cap, H))
        dec = ws.get("mlstm.decay_t", (T, H), f32, (cap, H))
        m = ws.get("mlstm.m", (T, H), f32, (cap, H))
        bias = self.params["gate_proj.bias"]
        ops.mlstm_gates(pre, bias[:H], bias[H:], self.cap, cache.tensors["m"], step.state_slots, step.seg_info,
                        len(step.segments), kf, dec, m)
        name, n_chunks, single, multi = self._step_lists
        tensors = step.extras["tensors"]
        carry = decay = None
        if multi:
            most = self.max_chunks(cap)
            carry = ws.get("mlstm.carry", (n_chunks, H, D, Dv + 1), f32, (most, H, D, Dv + 1))
            decay = ws.get("mlstm.decay", (n_chunks, H, D), f32, (most, H, D))
        o32 = ws.get("mlstm.o32", (T, H, Dv), f32, (cap, H, Dv))
        nq = ws.get("mlstm.nq", (T, H), f32, (cap, H))
        # q, k, v where the projection left them; the key factor, the head's decay, the normaliser's ones
        ops.gla_scan(proj[:, : H * D], proj[:, H * D: 2 * H * D], proj[:, 2 * H * D: self.g_row], None, None, 1.0,
                     D ** -0.5, cache.tensors["s"], step.state_slots, step.seg_info, len(step.segments), tensors[name],
                     n_chunks, tensors[name + ".segments"], single, multi, carry, decay, o32, k_fac=kf, a_head=dec,
                     ones_col=True, out_ones=nq)
        o = ws.get("mlstm.o", (T, H * Dv), dt, (cap, H * Dv))
        ops.mlstm_output(o32, nq, m, proj[:, self.g_row:], self.params["norm.weight"], self.eps, o)
        out = ws.get("mlstm.out", (T, self.hidden), dt, (cap, self.hidden))
        ops.linear(o, self.params["o_proj.weight"], out)
        return out
