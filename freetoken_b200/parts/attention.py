"""Grouped-query softmax attention over a paged cache.

Order of operations (python/freetoken/models/minimax_m3/attention.py:79-119): fused qkv
projection (rows q, k, v), per-head RMSNorm of q and k heads with one ``[head_dim]`` weight
each (:54-56,90-91), partial NeoX rotation of q and k (:92), keys and values of the new
tokens stored in the cache before it is read (python/freetoken/attention/triton.py:150),
causal softmax attention with scale ``head_dim^-0.5`` where query head ``h`` reads KV head
``h // group`` (python/freetoken/kernel/triton/attention.py:74,102,118-137), output
projection.  Norm, rotation and the page write are one kernel here; the projections are
library matrix products, as in the reference (python/freetoken/layers/linear.py:31-32).

Options beyond the reference's layer, all off by default: values of another size than the keys
(``v_head_dim``; both are padded with zeros to one size, a multiple of 16, in q and in the cache: a zero
column changes no score and gives a zero output column that the output projection never reads), a sink
in the softmax's denominator (``sink``: a logit that takes its share of the weights and has no value), an
output gate taken element by element from one more projection of the same input (``out_gate``), a layer
without keys and values of its own that reads the cache of an earlier layer (``own_kv=False``; the
schedule entry names the owner) and a cache that outlives the layer's own window because such readers
look farther back (``cache_window``), biases on the q, k and v projections (``proj_bias``), one learned sink
logit per head (``sink="learned"``), and a bias by the logarithm of the distance that is taken off the scaled score,
``r1_h ln(1 + r2_h (i - j))`` with two learned numbers per head (``log_dist_bias``; the kernels read it from a table
by distance that covers the engine's longest sequence, made in float64 and rounded once).
"""

from __future__ import annotations

from typing import Any, Dict, Optional, Tuple

import torch

from ..config.spec import PagedKVNeed, ParamSpec, PartSpec
from ..engine.attention_plan import DEAL_MOST_PIECES
from ..errors import ConfigError
from ..kernels import ops
from .base import MIXERS, BuildEnv, Mixer, StepState
from .rope import shared_position


TC_MIN_TOKENS = 128      # shortest step that goes to the tcgen05 attention kernel
TC_PAIR_MIN_TOKENS = 1024  # from this many tokens on, a step goes to the kernel with two query tiles per CTA
TC_PAIR_MIN_TOKENS_LONG = 256  # ... and from this many on when its longest request has TC_PAIR_MIN_SPAN keys and more
TC_PAIR_MIN_SPAN = 16384       # (rounded up to 2^n): such tiles are cut along the keys into enough pieces for every SM
TC_MIN_DECODE_SPAN = 0   # decode steps go there from this length of the longest request (rounded up to 2^n) on


def attention_kernel_form(dtype: torch.dtype, decode_only: bool = False, group: int = 1, n_tokens: int = 0,
                          head_dim: int = 0, page_size: int = 0, window: Optional[int] = None,
                          longest_span: int = 0, one_tile_only: bool = False, no_few: bool = False) -> Tuple[int, bool]:
    """``(query rows one attention CTA handles, the tcgen05 kernel's form for few rows)``.

    16 rows in the 32-bit kernel.  bfloat16 steps whose sizes the tcgen05 kernels take: 128 rows for
    long steps (``TC_MIN_TOKENS`` tokens and more; 256, two such tiles per CTA, from
    ``TC_PAIR_MIN_TOKENS`` tokens on, or from ``TC_PAIR_MIN_TOKENS_LONG`` for portions of long prompts: the
    rule for callers without a step's work lists; a step itself takes, from ``TC_PAIR_MIN_TOKENS_LONG`` tokens
    on, the form whose work list is estimated to end sooner, see ``GQAttention.prepare``);
    decode steps go to the same kernel in its form for tiles of at
    most 16 rows, where one warp takes the softmax (groups of up to 16 heads; ``longest_span`` is the longest
    request's length rounded up to a power of two, from which on they go there:
    ``TC_MIN_DECODE_SPAN``), larger groups to the 128-row kernel.  Otherwise 16 rows for decode steps
    of small groups and 64 in the bfloat16 mma.sync kernels.  ``one_tile_only``: of the tcgen05 kernels only
    the ones with a single query tile a piece may be chosen (they are the ones that take a bias by distance);
    ``no_few``: nor the form for tiles of at most 16 rows (a window or a sink: the 128-row form alone takes them)."""
    if dtype != torch.bfloat16:
        return 16, False
    sized = bool(head_dim and page_size)
    if window is not None:  # (of the tcgen05 kernels the one with a single 128-row tile a piece takes a window)
        one_tile_only = no_few = True
    if decode_only:
        if sized and not no_few and longest_span >= TC_MIN_DECODE_SPAN:
            if ops.attention_tc_few_fits(head_dim, page_size, group):
                return 16, True
            if ops.attention_tc_fits(head_dim, page_size, group):
                return 128, False
        return (16 if group <= 16 else 64), False
    tc = sized and ops.attention_tc_fits(head_dim, page_size, group)
    if tc and not one_tile_only and (n_tokens >= TC_PAIR_MIN_TOKENS or
               (n_tokens >= TC_PAIR_MIN_TOKENS_LONG and longest_span >= TC_PAIR_MIN_SPAN)):
        return 256, False
    if tc and n_tokens >= TC_MIN_TOKENS:
        return 128, False
    return 64, False


def attention_tile_rows(dtype: torch.dtype, decode_only: bool = False, group: int = 1, n_tokens: int = 0,
                        head_dim: int = 0, page_size: int = 0, window: Optional[int] = None,
                        longest_span: int = 0) -> int:
    """Query rows (tokens x group heads) one attention CTA handles (see :func:`attention_kernel_form`)."""
    return attention_kernel_form(dtype, decode_only, group, n_tokens, head_dim, page_size, window, longest_span)[0]


@MIXERS.register("gqa_attention")
class GQAttention(Mixer):
    """params: ``hidden``, ``n_heads``, ``n_kv_heads``, ``head_dim``, ``qk_norm`` (bool),
    ``eps``, ``gemma`` (bool), ``position`` (PartSpec of a position encoding), ``window``
    (None or tokens), ``scale`` (None = head_dim^-0.5); ``v_head_dim`` (head_dim), ``sink`` (None, a
    logit, or "learned": a tensor of one logit per head), ``proj_bias`` (bool), ``log_dist_bias`` (bool), ``out_gate`` (None | "sigmoid" | "silu"), ``own_kv`` (True), ``cache_window`` (how long the
    cache keeps a token: ``window``, or more, or None for ever, when other layers read it), ``init_std``."""

    graph_safe = True  # running a step twice writes the same keys and values again

    def __init__(self, spec: PartSpec, env: BuildEnv):
        super().__init__(spec, env)
        self.hidden = int(spec["hidden"])
        self.n_heads = int(spec["n_heads"])
        self.n_kv_heads = int(spec["n_kv_heads"])
        self.head_dim = int(spec["head_dim"])
        if self.n_heads % self.n_kv_heads:
            raise ConfigError("gqa_attention: n_heads must be a multiple of n_kv_heads")
        self.v_dim = int(spec.get("v_head_dim") or self.head_dim)
        if not 1 <= self.head_dim <= 256 or not 1 <= self.v_dim <= 256:
            raise ConfigError(
                f"gqa_attention: head sizes {self.head_dim} (keys) and {self.v_dim} (values) must be in [1, 256]")
        self.pad_dim = -(-max(self.head_dim, self.v_dim) // 16) * 16  # what the attention kernels take
        self.padded = self.pad_dim != self.head_dim or self.pad_dim != self.v_dim
        self.group = self.n_heads // self.n_kv_heads
        self.qk_norm = bool(spec.get("qk_norm", True))
        self.eps = float(spec.get("eps", 1e-6))
        self.gemma = bool(spec.get("gemma", True))
        self.window: Optional[int] = spec.get("window")
        self.cache_window: Optional[int] = spec["cache_window"] if "cache_window" in spec.params else self.window
        if self.window is not None and self.window < 1:
            raise ConfigError("gqa_attention: a window holds at least the token itself")
        if self.cache_window is not None and (self.window is None or self.cache_window < self.window):
            raise ConfigError("gqa_attention: the cache must keep a token at least as long as the layer's window")
        self.learned_sink = spec.get("sink") == "learned"
        self.sink: Optional[float] = None if spec.get("sink") is None or self.learned_sink else float(spec["sink"])
        self.proj_bias = bool(spec.get("proj_bias", False))
        self.log_dist_bias = bool(spec.get("log_dist_bias", False))
        self._dist_table: Optional[torch.Tensor] = None
        self.out_gate: Optional[str] = spec.get("out_gate")
        if self.out_gate not in (None, "sigmoid", "silu"):
            raise ConfigError(f"gqa_attention: unknown output gate '{self.out_gate}'")
        self.own_kv = bool(spec.get("own_kv", True))
        self.scale = float(spec.get("scale") or self.head_dim ** -0.5)
        self.position = shared_position(spec.get("position") or PartSpec("none"), env)
        self.rotary_dim = int(getattr(self.position, "rotary_dim", 0))
        if self.rotary_dim > self.head_dim:
            raise ConfigError("gqa_attention: rotary_dim exceeds head_dim")
        # more query heads per KV head than the kernels' tiles have rows: every KV head is taken as `kv_split` heads of
        # the same keys (the smallest split that fits), and the work is planned for that many heads
        most = attention_tile_rows(env.dtype) if env.dtype != torch.bfloat16 else 64
        self.kv_split = next(s for s in range(1, self.group + 1) if self.group % s == 0 and self.group // s <= most)
        self.plan_group = self.group // self.kv_split
        self.plan_kv_heads = self.n_kv_heads * self.kv_split
        self.q_dim = self.n_heads * self.head_dim
        self.kv_dim = self.n_kv_heads * self.head_dim
        self.vv_dim = self.n_kv_heads * self.v_dim
        self.o_dim = self.n_heads * self.v_dim
        self.gate_dim = self.o_dim if self.out_gate else 0
        # rows of the one projection: q, then (a layer with keys and values of its own) k and v, then the gate
        self.k_row = self.q_dim
        self.v_row = self.k_row + (self.kv_dim if self.own_kv else 0)
        self.g_row = self.v_row + (self.vv_dim if self.own_kv else 0)
        self.proj_rows = self.g_row + self.gate_dim
        self.plain = not (self.padded or self.sink is not None or self.out_gate or self.kv_split > 1 or not self.own_kv
                          or self.learned_sink or self.proj_bias or self.log_dist_bias)
        self._o_weight: Optional[torch.Tensor] = None

    # ------------------------------------------------------------------ tensors
    def param_specs(self) -> Dict[str, ParamSpec]:
        std = self.spec.get("init_std")  # spread of random weights: (projections of the input, output projection)
        std_in, std_out = (float(std[0]), float(std[1])) if std else (0.02, 0.02)
        out = {
            "qkv_proj.weight": ParamSpec((self.proj_rows, self.hidden), init=("normal", 0.0, std_in)),
            "o_proj.weight": ParamSpec((self.hidden, self.o_dim), init=("normal", 0.0, std_out)),
        }
        if self.qk_norm:
            init = ("normal", 0.0, 0.02) if self.gemma else ("normal", 1.0, 0.02)
            if std:
                init = (init[0], init[1], 0.2)
            out["q_norm.weight"] = ParamSpec((self.head_dim,), "float32", init, store="bfloat16")
            if self.own_kv:
                out["k_norm.weight"] = ParamSpec((self.head_dim,), "float32", init, store="bfloat16")
        f32 = dict(dtype="float32", store="bfloat16")
        if self.proj_bias:
            out["q_bias"] = ParamSpec((self.q_dim,), init=("normal", 0.0, 0.3 if std else 0.02), **f32)
            if self.own_kv:
                out["k_bias"] = ParamSpec((self.kv_dim,), init=("normal", 0.0, 0.3 if std else 0.02), **f32)
                out["v_bias"] = ParamSpec((self.vv_dim,), init=("normal", 0.0, 0.3 if std else 0.02), **f32)
        if self.learned_sink:
            out["sink"] = ParamSpec((self.n_heads,), init=("normal", 0.0, 1.0 if std else 0.02), **f32)
        if self.log_dist_bias:
            out["r1"] = ParamSpec((self.n_heads,), init=("normal", 0.5 if std else 0.0, 0.2 if std else 0.02), **f32)
            out["r2"] = ParamSpec((self.n_heads,), init=("uniform", 0.05, 1.0), **f32)
        return out

    def dist_table(self) -> Optional[torch.Tensor]:
        """``[heads, longest sequence]``: what distance ``d`` adds to a head's scaled scores, ``-r1 ln(1 + r2 d)``;
        made at the first call, when the engine's longest sequence is settled."""
        if not self.log_dist_bias:
            return None
        if self._dist_table is None:
            r1, r2 = self.params["r1"].double()[:, None], self.params["r2"].double()[:, None]
            d = torch.arange(max(1, int(self.env.max_seq_len)), dtype=torch.float64, device=r1.device)[None, :]
            self._dist_table = (-r1 * torch.log1p(r2 * d)).float().contiguous()
        return self._dist_table

    def bind(self, tensors) -> None:
        super().bind(tensors)
        w = self.params["o_proj.weight"]
        if self.pad_dim != self.v_dim:  # zero columns where the attention output has its padding
            wp = torch.zeros((self.hidden, self.n_heads, self.pad_dim), dtype=w.dtype, device=w.device)
            wp[:, :, : self.v_dim] = w.view(self.hidden, self.n_heads, self.v_dim)
            w = wp.view(self.hidden, self.n_heads * self.pad_dim)
        self._o_weight = w
        self._dist_table = None

    def cache_need(self):
        if not self.own_kv:
            return None
        return PagedKVNeed((("k", self.n_kv_heads, self.pad_dim),
                            ("v", self.n_kv_heads, self.pad_dim)), self.cache_window)

    def workspace_bytes(self, n_tokens: int) -> int:
        item = 4 if self.env.dtype == torch.float32 else 2
        # qkv, q, o, out; and the 32-bit partial results of tiles split along the keys (at most
        # attention_plan.DEAL_MOST_PIECES pieces per SM, 256 rows each at most)
        rows = n_tokens * (self.proj_rows + self.vv_dim + 2 * self.n_heads * self.pad_dim + self.hidden) * item
        return rows + DEAL_MOST_PIECES * 148 * 256 * (self.pad_dim + 2) * 4

    # ------------------------------------------------------------------ step
    def kernel_form(self, decode_only: bool, n_tokens: int = 0, page_size: int = 0, longest_span: int = 0):
        # (the tcgen05 kernels take no split KV heads; a sink or a window goes with the 128-row form alone)
        sized = self.kv_split == 1
        has_sink = self.sink is not None or self.learned_sink
        special = has_sink or self.window is not None
        return attention_kernel_form(self.env.dtype, decode_only, self.plan_group, n_tokens,
                                     self.pad_dim if sized else 0, page_size, self.window, longest_span,
                                     one_tile_only=special or self.log_dist_bias, no_few=special)

    def tile_rows(self, decode_only: bool, n_tokens: int = 0, page_size: int = 0, longest_span: int = 0) -> int:
        return self.kernel_form(decode_only, n_tokens, page_size, longest_span)[0]

    def plan_key(self, decode_only: bool = False, n_tokens: int = 0, page_size: int = 0, longest_span: int = 0):
        rows, few_rows = self.kernel_form(decode_only, n_tokens, page_size, longest_span)
        return ("attention", self.plan_group, rows, self.window, self.plan_kv_heads, self.pad_dim, few_rows)

    def prepare(self, builder) -> None:
        """Ask the step for the work list this mixer's attention kernel runs from."""
        n_tokens = sum(q for q, _ in builder.seg_lens)
        page_size = builder.engine.config.page_size if builder.engine is not None else 0
        # forward() of the same step runs the kernel this work list was made for
        rows, few_rows = self.kernel_form(builder.decode_only, n_tokens, page_size, builder.longest_span())
        if rows >= 128 and not few_rows and not builder.decode_only and n_tokens >= TC_PAIR_MIN_TOKENS_LONG \
                and self.sink is None and not self.learned_sink and not self.log_dist_bias and self.window is None \
                and hasattr(builder, "cheaper_attention_rows"):
            # one or two query tiles a piece: whichever work list the kernel is estimated to get through sooner
            rows = builder.cheaper_attention_rows(self.plan_group, self.window, self.plan_kv_heads, self.pad_dim)
        self._step_plan = builder.attention_plan(self.plan_group, rows, self.window, self.plan_kv_heads, self.pad_dim,
                                                 few_rows)

    def forward(self, h: torch.Tensor, step: StepState, cache: Any, writes_cache: bool) -> torch.Tensor:
        if not self.plain:
            return self._forward_with_options(h, step, cache, writes_cache)
        T = h.shape[0]
        ws, dt = self.env.workspace, self.env.dtype
        cap = self.env.max_step_tokens
        n_proj = self.q_dim + (2 * self.kv_dim if writes_cache else 0)
        qkv = ws.get("attn.qkv", (T, n_proj), dt, (cap, self.q_dim + 2 * self.kv_dim))
        w = self.params["qkv_proj.weight"]
        ops.linear(h, w if writes_cache else w[: self.q_dim], qkv)
        q = ws.get("attn.q", (T, self.n_heads, self.head_dim), dt, (cap, self.n_heads, self.head_dim))
        sections = [dict(first_head=0, n_heads=self.n_heads,
                         norm_weight=self.params.get("q_norm.weight"), rotate=True, dense_out=q)]
        if writes_cache:
            sections.append(dict(first_head=self.n_heads, n_heads=self.n_kv_heads,
                                 norm_weight=self.params.get("k_norm.weight"), rotate=True,
                                 slab=cache.slabs["k"], slot_map=cache.slot_map))
            sections.append(dict(first_head=self.n_heads + self.n_kv_heads, n_heads=self.n_kv_heads,
                                 norm_weight=None, rotate=False,
                                 slab=cache.slabs["v"], slot_map=cache.slot_map))
        ops.norm_rope_store(qkv, self.head_dim, self.rotary_dim, step.positions,
                            self.position.table(), self.eps, self.gemma, sections)
        plan = step.attention_plans[self._step_plan]
        o = ws.get("attn.o", (T, self.n_heads, self.head_dim), dt, (cap, self.n_heads, self.head_dim))
        ops.paged_attention(q, cache.slabs["k"], cache.slabs["v"], cache.block_table, step.seg_info,
                            len(step.segments), plan.items_dev, plan.n_items, plan.part_o, plan.part_ml,
                            o, self._step_plan[2], self.scale, self.window, few_rows=self._step_plan[6])
        out = ws.get("attn.out", (T, self.hidden), dt, (cap, self.hidden))
        ops.linear(o.view(T, self.q_dim), self.params["o_proj.weight"], out)
        return out

    def _forward_with_options(self, h: torch.Tensor, step: StepState, cache: Any, writes_cache: bool) -> torch.Tensor:
        """The same order of operations with padded heads, values of their own size, a sink, an output gate, split
        KV heads, or another layer's keys and values."""
        if writes_cache != self.own_kv:
            raise ConfigError("gqa_attention: a layer with keys and values of its own owns its cache, and only such a layer")
        T = h.shape[0]
        ws, dt, cap = self.env.workspace, self.env.dtype, self.env.max_step_tokens
        D, Dv, Dp, H, G = self.head_dim, self.v_dim, self.pad_dim, self.n_heads, self.n_kv_heads
        proj = ws.get("attn.proj", (T, self.proj_rows), dt, (cap, self.proj_rows))
        ops.linear(h, self.params["qkv_proj.weight"], proj)
        q = ws.get("attn.q", (T, H, Dp), dt, (cap, H, Dp))
        sections = [dict(first_head=0, n_heads=H, norm_weight=self.params.get("q_norm.weight"), rotate=True,
                         dense_out=q, dst_head_dim=Dp, bias=self.params.get("q_bias"))]
        v_too = self.own_kv and Dv == D  # the value heads then lie on the same grid of heads as q and k
        if self.own_kv:
            sections.append(dict(first_head=H, n_heads=G, norm_weight=self.params.get("k_norm.weight"), rotate=True,
                                 slab=cache.slabs["k"], slot_map=cache.slot_map, dst_head_dim=Dp,
                                 bias=self.params.get("k_bias")))
            if v_too:
                sections.append(dict(first_head=H + G, n_heads=G, norm_weight=None, rotate=False,
                                     slab=cache.slabs["v"], slot_map=cache.slot_map, dst_head_dim=Dp,
                                     bias=self.params.get("v_bias")))
        ops.norm_rope_store(proj, D, self.rotary_dim, step.positions, self.position.table(), self.eps, self.gemma,
                            sections)
        if self.own_kv and not v_too:  # values of another size: a pass of their own over a copy of their columns
            v = ws.get("attn.v", (T, self.vv_dim), dt, (cap, self.vv_dim))
            v.copy_(proj[:, self.v_row: self.g_row])
            ops.norm_rope_store(v, Dv, 0, step.positions, None, self.eps, self.gemma,
                                [dict(first_head=0, n_heads=G, norm_weight=None, rotate=False, slab=cache.slabs["v"],
                                      slot_map=cache.slot_map, dst_head_dim=Dp, bias=self.params.get("v_bias"))])
        plan = step.attention_plans[self._step_plan]
        o = ws.get("attn.o", (T, H, Dp), dt, (cap, H, Dp))
        ops.paged_attention(q, cache.slabs["k"], cache.slabs["v"], cache.block_table, step.seg_info,
                            len(step.segments), plan.items_dev, plan.n_items, plan.part_o, plan.part_ml,
                            o, self._step_plan[2], self.scale, self.window, few_rows=self._step_plan[6],
                            kv_split=self.kv_split, sink=self.params["sink"] if self.learned_sink else self.sink,
                            dist_bias=self.dist_table())
        if self.out_gate:
            ops.gated_heads(o, proj[:, self.g_row:], o, Dv, self.out_gate)
        out = ws.get("attn.out", (T, self.hidden), dt, (cap, self.hidden))
        ops.linear(o.view(T, H * Dp), self._o_weight, out)
        return out
