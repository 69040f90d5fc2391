"""Norms with the residual sum fused in: RMSNorm (plain or Gemma form) and Dynamic Tanh.

``y = x * rsqrt(mean(x^2) + eps) * (1 + w)`` in 32-bit (python/freetoken/kernel/triton/norm.py:65-75;
``1 + w`` only in the Gemma form, :69-72); the fused variant first adds the sub-layer output
to the residual stream (:101-112, python/freetoken/layers/norm.py:120-147).  The residual
stream itself is kept in 32-bit here, so the sum is never rounded.

``dynamic_tanh``: ``y = tanh(alpha z) w + b`` with a learned scalar ``alpha``; it takes no mean and no
variance of the row, so it has no ``eps``.  Its fused form takes everything a :class:`StreamSum` holds.
"""

from __future__ import annotations

from typing import Dict, Optional

import torch

from ..config.spec import ParamSpec, PartSpec
from ..kernels import ops
from .base import NORMS, BuildEnv, Norm, NormedSum, RouteSum, StreamSum


@NORMS.register("rmsnorm")
class RMSNorm(Norm):
    """params: ``size``, ``eps``, ``gemma`` (bool: multiply by ``1 + w``), ``scalar`` (bool: the weight is one
    number for all coordinates; the checkpoint tensor has no axis)."""

    takes_route_sum = True
    takes_normed_sum = True

    def __init__(self, spec: PartSpec, env: BuildEnv):
        super().__init__(spec, env)
        self.size = int(spec["size"])
        self.eps = float(spec["eps"])
        self.gemma = bool(spec.get("gemma", True))
        self.scalar = bool(spec.get("scalar", False))

    def param_specs(self) -> Dict[str, ParamSpec]:
        init = ("normal", 0.0, 0.02) if self.gemma else ("normal", 1.0, 0.02)
        if self.scalar and self.spec.get("init_std") is not None:
            init = (init[0], init[1], float(self.spec["init_std"]))
        return {"weight": ParamSpec(() if self.scalar else (self.size,), "float32", init, store="bfloat16")}

    def bind(self, tensors) -> None:
        super().bind(tensors)
        if self.scalar:  # the kernels take one weight per coordinate
            self.params["weight"] = self.params["weight"].reshape(1).expand(self.size).contiguous()

    def forward(self, x: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        ops.add_rmsnorm(x, None, self.params["weight"], self.eps, self.gemma, out)
        return out

    def add_forward(self, x: Optional[torch.Tensor], residual: torch.Tensor, out: torch.Tensor,
                    out_f32: Optional[torch.Tensor] = None,
                    rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        if isinstance(x, StreamSum):
            x.fold(residual)
            x = None
        if isinstance(x, NormedSum):  # the sub-layer's own norm, the sum and this norm in one pass
            data, routed = x.kernel_args()
            ops.postnorm_add_norm(data, routed, x.norm.params["weight"], x.norm.eps, x.norm.gemma, residual,
                                  self.params["weight"], self.eps, self.gemma, out, out_f32=out_f32, rows=rows)
            return out
        if isinstance(x, RouteSum):
            ops.add_rmsnorm_routes(x.y, x.pos, x.top_k, x.shared, residual, self.params["weight"], self.eps,
                                   self.gemma, out, out_f32=out_f32, rows=rows)
        else:
            ops.add_rmsnorm(x, residual, self.params["weight"], self.eps, self.gemma, out,
                            out_f32=out_f32, rows=rows)
        return out


@NORMS.register("dynamic_tanh")
class DynamicTanh(Norm):
    """params: ``size``.  Tensors: ``weight [size]``, ``bias [size]``, ``alpha []``, all 32-bit."""

    takes_route_sum = True
    takes_stream_sum = True

    def __init__(self, spec: PartSpec, env: BuildEnv):
        super().__init__(spec, env)
        self.size = int(spec["size"])

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {"weight": ParamSpec((self.size,), "float32", ("normal", 1.0, 0.1), store="bfloat16"),
                "bias": ParamSpec((self.size,), "float32", ("normal", 0.0, 0.1), store="bfloat16"),
                "alpha": ParamSpec((), "float32", ("normal", 0.5, 0.05), store="bfloat16")}

    def bind(self, tensors) -> None:
        super().bind(tensors)
        self._norm = ("dynamic_tanh", self.params["weight"], self.params["bias"], self.params["alpha"].reshape(1))

    def forward(self, x: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        ops.stream_add_norm(None, out, x1=x, norm=self._norm)
        return out

    def add_forward(self, x, residual: torch.Tensor, out: torch.Tensor,
                    out_f32: Optional[torch.Tensor] = None,
                    rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        if out_f32 is not None:
            raise NotImplementedError("dynamic_tanh: no 32-bit copy of the output")
        args = StreamSum.of(x).kernel_args(residual) if x is not None else {}
        ops.stream_add_norm(residual, out, norm=self._norm, rows=rows, **args)
        return out
