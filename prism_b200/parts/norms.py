"""Norm parts.  ``rmsnorm``: andre-fu/prism's ``fused_rms_norm``
(engine/fused_kernels.py:30-65) with the residual add that precedes it
(engine/executor.py:122-124) fused in, eps and width as parameters."""

from __future__ import annotations

from .base import Norm, ParamSpec, WeightSource, register_part
from .. import ops


@register_part("norm", "rmsnorm")
class RMSNorm(Norm):
    """``x * rsqrt(mean(x^2) + eps) * weight``: the weight multiplies (no
    ``1 + w``), no bias, no mean subtraction (fused_kernels.py:41-49)."""

    def __init__(self, width: int, eps: float):
        self.width = int(width)
        self.eps = float(eps)

    def params(self):
        return [ParamSpec("weight", (WeightSource("weight", (self.width,), "norm"),))]

    def forward(self, ctx, residual, delta, rows=None):
        n = residual.shape[0] if rows is None else rows.shape[0]
        out = ctx.alloc((n, self.width), ctx.dtype)
        ops.add_rmsnorm(residual, delta, self.w["weight"], self.eps, out, rows)
        return out
