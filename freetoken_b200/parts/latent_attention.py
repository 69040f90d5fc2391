"""Latent attention: queries, keys and values through low-rank latents, one rotated key part for all heads.

Per token, with ``H`` heads of ``dim`` unrotated and ``rot_dim`` rotated query/key dimensions, values of
``v_head_dim``, a key/value latent of ``kv_rank`` and a query latent of ``q_rank``::

    c_q = RMSnorm(W_dq h)                       q_h = W_uq,h c_q = [q_flat,h | q_rot,h]
    [c_pre | k_rot] = W_dkv h                   c = RMSnorm(c_pre);  k_rot is turned by the position, as q_rot,h is
    score_h(i, j) = (q_flat,h(i) . (W_uk,h c(j)) + q_rot,h(i) . k_rot(j)) * scale
    out_h(i) = sum_j weight_h(i, j) W_uv,h c(j)

Only ``c`` and the turned ``k_rot`` are cached, one row ``[c | k_rot | zeros]`` per token, and the keys and
values are never built: ``q_flat,h . (W_uk,h c) = (W_uk,h^T q_flat,h) . c``, so the query is taken into the
latent space (a product per head) and attention runs as one KV head of size ``kv_rank + rot_dim`` under all
``H`` query heads, with the cache row as key *and* value; the weighted sum of latents then goes through
``W_uv,h`` (a product per head) and the output projection.  The attention kernels are the framework's own
(:func:`ops.paged_attention` with one slab for keys and values); sliding window, a learned sink per head in the
softmax's denominator and the scale are their options.  Norms, rotation and softmax are 32-bit.

Without a query latent (``q_rank = None``) the queries are a plain projection of the input, ``q_h = W_q,h h``.  With
``head_gate`` every head's output is multiplied by ``sigmoid(w_g,h . h)``, one logit per head from one more row of
the input projection.

``kv_rank + rot_dim`` may be at most 256 (the attention kernels' largest head); the tcgen05 kernels take it
when it is 128.  The reference has no such layer.
"""

from __future__ import annotations

from typing import Any, Dict, Optional

import torch

from ..config.spec import PagedKVNeed, ParamSpec, PartSpec
from ..engine.attention_plan import DEAL_MOST_PIECES
from ..errors import ConfigError
from ..kernels import ops
from .attention import attention_kernel_form
from .base import MIXERS, BuildEnv, Mixer, StepState
from .rope import shared_position


@MIXERS.register("latent_attention")
class LatentAttention(Mixer):
    """params: ``hidden``, ``n_heads``, ``head_dim`` (unrotated), ``rot_dim`` (rotated, one key part for all heads),
    ``v_head_dim``, ``q_rank`` (None: no query latent), ``kv_rank``, ``head_gate`` (bool), ``eps`` (of the latents' norms), ``position`` (PartSpec of a rotary
    encoding whose ``rotary_dim <= rot_dim``), ``window`` (None or tokens), ``scale`` (None = (head_dim +
    rot_dim)^-0.5), ``sink`` (None | "learned": one logit per head), ``init_std``."""

    graph_safe = True  # running a step twice writes the same cache rows again

    def __init__(self, spec: PartSpec, env: BuildEnv):
        super().__init__(spec, env)
        g = lambda k: int(spec[k])  # noqa: E731
        self.hidden, self.n_heads, self.head_dim, self.rot_dim = g("hidden"), g("n_heads"), g("head_dim"), g("rot_dim")
        self.v_dim, self.kv_rank = g("v_head_dim"), g("kv_rank")
        self.q_latent = spec.get("q_rank") is not None
        self.q_rank = g("q_rank") if self.q_latent else 0
        self.head_gate = bool(spec.get("head_gate", False))
        if min(self.hidden, self.n_heads, self.head_dim, self.v_dim, self.kv_rank) < 1 or self.rot_dim < 0 \
                or (self.q_latent and self.q_rank < 1):
            raise ConfigError("latent_attention: sizes must be positive")
        self.key_dim = self.kv_rank + self.rot_dim
        if self.key_dim > 256:
            raise ConfigError(f"latent_attention: kv_rank + rot_dim = {self.key_dim} exceeds 256, the attention "
                              "kernels' largest head")
        self.pad_dim = -(-self.key_dim // 16) * 16
        self.eps = float(spec.get("eps", 1e-6))
        self.window: Optional[int] = spec.get("window")
        if self.window is not None and self.window < 1:
            raise ConfigError("latent_attention: a window holds at least the token itself")
        self.scale = float(spec.get("scale") or (self.head_dim + self.rot_dim) ** -0.5)
        self.sink = spec.get("sink")
        if self.sink not in (None, "learned"):
            raise ConfigError(f"latent_attention: unknown sink '{self.sink}'")
        self.position = shared_position(spec.get("position") or PartSpec("none"), env)
        self.n_rot = int(getattr(self.position, "rotary_dim", 0))
        self.interleaved = bool(getattr(self.position, "interleaved", False))
        if self.n_rot > self.rot_dim:
            raise ConfigError("latent_attention: more rotated dimensions than the rotated part has")
        self.q_dim = self.head_dim + self.rot_dim
        # rows of the input projection: [query latent |] key/value latent | rotated key part [| a gate logit per head]
        self.lat_rows = self.q_rank + self.kv_rank + self.rot_dim
        self.in_rows = self.lat_rows + (self.n_heads if self.head_gate else 0)
        most = 16 if env.dtype != torch.bfloat16 else 64  # query heads on the one KV head that a tile's rows take
        self.kv_split = next(s for s in range(1, self.n_heads + 1) if self.n_heads % s == 0 and self.n_heads // s <= most)
        self.plan_group = self.n_heads // self.kv_split
        self._w_uk: Optional[torch.Tensor] = None
        self._w_uv: Optional[torch.Tensor] = None

    # ------------------------------------------------------------------ tensors
    def param_specs(self) -> Dict[str, ParamSpec]:
        std = self.spec.get("init_std")
        s_in, s_q, s_kv, s_out = (tuple(float(x) for x in std) if std else (0.02,) * 4)
        H = self.n_heads
        out = {
            "in_proj.weight": ParamSpec((self.in_rows, self.hidden), init=("normal", 0.0, s_in)),
            "kv_norm.weight": ParamSpec((self.kv_rank,), "float32", ("normal", 1.0, 0.2 if std else 0.02), store="bfloat16"),
            "q_up.weight": ParamSpec((H * self.q_dim, self.q_rank if self.q_latent else self.hidden),
                                     init=("normal", 0.0, s_q if self.q_latent else s_in)),
            "k_up.weight": ParamSpec((H * self.head_dim, self.kv_rank), init=("normal", 0.0, s_kv)),
            "v_up.weight": ParamSpec((H * self.v_dim, self.kv_rank), init=("normal", 0.0, s_kv)),
            "o_proj.weight": ParamSpec((self.hidden, H * self.v_dim), init=("normal", 0.0, s_out)),
        }
        if self.q_latent:
            out["q_norm.weight"] = ParamSpec((self.q_rank,), "float32", ("normal", 1.0, 0.2 if std else 0.02), store="bfloat16")
        if self.sink == "learned":
            out["sink"] = ParamSpec((H,), "float32", ("normal", 0.0, 1.0 if std else 0.02), store="bfloat16")
        return out

    def bind(self, tensors) -> None:
        super().bind(tensors)
        H = self.n_heads
        # per head: [dim, kv_rank] takes a query into the latent space, [kv_rank, vdim] a latent sum to values
        self._w_uk = self.params["k_up.weight"].view(H, self.head_dim, self.kv_rank).contiguous()
        self._w_uv = self.params["v_up.weight"].view(H, self.v_dim, self.kv_rank).transpose(1, 2).contiguous()

    def cache_need(self):
        return PagedKVNeed((("kv", 1, self.pad_dim),), self.window)

    def workspace_bytes(self, n_tokens: int) -> int:
        item = 4 if self.env.dtype == torch.float32 else 2
        H = self.n_heads
        rows = n_tokens * (self.in_rows + self.q_rank + H * (self.q_dim + 2 * self.pad_dim + self.v_dim) + self.hidden) * item
        return rows + DEAL_MOST_PIECES * 148 * 256 * (self.pad_dim + 2) * 4

    # ------------------------------------------------------------------ step
    def kernel_form(self, decode_only: bool, n_tokens: int = 0, page_size: int = 0, longest_span: int = 0):
        # (keys that are the values, a window and a sink together: the tiles of 16 / 64 rows take them, and of the
        # tcgen05 kernels the one with a single 128-row tile a piece, whose head is 128 wide)
        sized = self.kv_split == 1
        return attention_kernel_form(self.env.dtype, decode_only, self.plan_group, n_tokens, self.pad_dim if sized else 0,
                                     page_size, self.window, longest_span, one_tile_only=True, no_few=True)

    def plan_key(self, decode_only: bool = False, n_tokens: int = 0, page_size: int = 0, longest_span: int = 0):
        rows, few = self.kernel_form(decode_only, n_tokens, page_size, longest_span)
        return ("attention", self.plan_group, rows, self.window, self.kv_split, self.pad_dim, few)

    def prepare(self, builder) -> None:
        n_tokens = sum(q for q, _ in builder.seg_lens)
        page_size = builder.engine.config.page_size if builder.engine is not None else 0
        rows, few = self.kernel_form(builder.decode_only, n_tokens, page_size, builder.longest_span())
        self._step_plan = builder.attention_plan(self.plan_group, rows, self.window, self.kv_split, self.pad_dim, few)

    def forward(self, h: torch.Tensor, step: StepState, cache: Any, writes_cache: bool) -> torch.Tensor:
        if not writes_cache:
            raise ConfigError("latent_attention: the layer owns its cache")
        T = h.shape[0]
        ws, dt, cap = self.env.workspace, self.env.dtype, self.env.max_step_tokens
        H, D, R, Dv, C, P = self.n_heads, self.head_dim, self.rot_dim, self.v_dim, self.kv_rank, self.pad_dim
        proj = ws.get("latent.proj", (T, self.in_rows), dt, (cap, self.in_rows))
        ops.linear(h, self.params["in_proj.weight"], proj)
        cq = ws.get("latent.cq", (T, self.q_rank), dt, (cap, self.q_rank))
        slab = cache.slabs["kv"]
        table = self.position.table()
        ops.latent_store(proj[:, : self.lat_rows], self.q_rank, C, R, self.n_rot, self.interleaved,
                         self.params.get("q_norm.weight"), self.params["kv_norm.weight"], self.eps, step.positions, table,
                         cq, slab, cache.slot_map)
        q = ws.get("latent.q", (T, H, self.q_dim), dt, (cap, H, self.q_dim))
        ops.linear(cq if self.q_latent else h, self.params["q_up.weight"], q.view(T, H * self.q_dim))
        qa = ws.get("latent.q_abs", (T, H, P), dt, (cap, H, P))
        ops.heads_linear(q[:, :, :D], self._w_uk, qa[:, :, :C])
        ops.latent_query_rotate(q, D, R, self.n_rot, self.interleaved, step.positions, table, qa, C)
        plan = step.attention_plans[self._step_plan]
        o = ws.get("latent.o", (T, H, P), dt, (cap, H, P))
        ops.paged_attention(qa, slab, slab, cache.block_table, step.seg_info, len(step.segments), plan.items_dev,
                            plan.n_items, plan.part_o, plan.part_ml, o, self._step_plan[2], self.scale, self.window,
                            few_rows=self._step_plan[6], kv_split=self.kv_split, sink=self.params.get("sink"))
        ov = ws.get("latent.ov", (T, H, Dv), dt, (cap, H, Dv))
        ops.heads_linear(o[:, :, :C], self._w_uv, ov)
        if self.head_gate:
            ops.head_gate(ov, proj[:, self.lat_rows:])
        out = ws.get("latent.out", (T, self.hidden), dt, (cap, self.hidden))
        ops.linear(ov.view(T, H * Dv), self.params["o_proj.weight"], out)
        return out
