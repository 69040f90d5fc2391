"""Several mixers side by side on one input, their results normed and averaged.

``out = (1 / n) sum_i unit(mixer_i(h)) * w_i`` with ``unit`` the division of a row by its root mean square over the
model width and one plain weight vector per branch (``<name>.out``); the mixers' own tensors lie under their
names.  Each branch keeps what it keeps (pages, a state slot): the part hands the cache manager all their needs
and every branch gets the view of its own.  The reference has no such layer.
"""

from __future__ import annotations

from typing import Any, Dict, List, Tuple

import torch

from ..config.spec import ParamSpec, PartSpec
from ..errors import ConfigError
from ..kernels import ops
from .base import MIXERS, BuildEnv, Mixer, Part, StepState, as_rows


@MIXERS.register("side_by_side")
class SideBySide(Mixer):
    """params: ``hidden``, ``branches`` (a tuple of ``(name, PartSpec of a mixer)``, two to four), ``eps`` (of the
    branch norms), ``init_std``."""

    def __init__(self, spec: PartSpec, env: BuildEnv):
        super().__init__(spec, env)
        self.hidden = int(spec["hidden"])
        self.eps = float(spec.get("eps", 1e-6))
        pairs = list(spec["branches"])
        if not 1 <= len(pairs) <= 4:
            raise ConfigError("side_by_side: one to four branches")
        self.names: List[str] = [str(n) for n, _ in pairs]
        self.branches: List[Mixer] = [MIXERS.build(s, env) for _, s in pairs]
        self.graph_safe = all(getattr(b, "graph_safe", False) for b in self.branches)
        self.graph_recordable = all(getattr(b, "graph_safe", False) or getattr(b, "graph_recordable", False)
                                    for b in self.branches)

    def children(self) -> Dict[str, Part]:
        return dict(zip(self.names, self.branches))

    def param_specs(self) -> Dict[str, ParamSpec]:
        wide = self.spec.get("init_std") is not None
        return {f"{n}.out": ParamSpec((self.hidden,), "float32", ("normal", 1.0, 0.2 if wide else 0.02), store="bfloat16")
                for n in self.names}

    def cache_need(self) -> Tuple:
        """One need per branch (None where a branch keeps nothing): the engine gives a view for each."""
        return tuple(b.cache_need() for b in self.branches)

    def workspace_bytes(self, n_tokens: int) -> int:
        item = 4 if self.env.dtype == torch.float32 else 2
        return n_tokens * self.hidden * item

    def plan_key(self, *a, **kw):
        for b in self.branches:
            if hasattr(b, "plan_key"):
                return b.plan_key(*a, **kw)
        return ("side_by_side",)

    def prepare(self, builder) -> None:
        for b in self.branches:
            prep = getattr(b, "prepare", None)
            if prep is not None:
                prep(builder)

    def forward(self, h: torch.Tensor, step: StepState, cache: Any, writes_cache: bool) -> torch.Tensor:
        if not isinstance(cache, (tuple, list)) or len(cache) != len(self.branches):
            raise ConfigError("side_by_side: a cache view per branch is expected")
        T = h.shape[0]
        ws, dt, cap = self.env.workspace, self.env.dtype, self.env.max_step_tokens
        ys = [as_rows(b.forward(h, step, c, writes_cache)) for b, c in zip(self.branches, cache)]
        out = ws.get("side_by_side.out", (T, self.hidden), dt, (cap, self.hidden))
        ops.norm_mean(ys, [self.params[f"{n}.out"] for n in self.names], self.eps, out)
        return out
