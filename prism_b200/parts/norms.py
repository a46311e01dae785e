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

    def __init__(self, width: int, eps: float, tensor: str = "weight", optional: bool = False):
        self.width = int(width)
        self.eps = float(eps)
        self.tensor = tensor          # the weight's name in the model file, after the part's prefix
        self.optional = bool(optional)    # the model file may leave the weight out: the block then skips this norm

    def params(self):
        return [ParamSpec("weight", (WeightSource(self.tensor, (self.width,), "norm"),), optional=self.optional)]

    def forward(self, ctx, residual, delta, rows=None):
        n = residual.shape[0] if rows is None else rows.shape[0]
        out = ctx.alloc((n, self.width), ctx.dtype)
        ops.add_rmsnorm(residual, delta, self.w["weight"], self.eps, out, rows)
        return out

    def forward_post(self, ctx, x, delta, alpha: float = 1.0):
        """Norm after the sum: ``x <- rmsnorm(alpha * x + delta) * weight`` in place on the float32 rows; returns
        the new rows in the compute dtype (``x`` itself in a float32 engine)."""
        copy = None if ctx.dtype == ops.torch.float32 else ctx.alloc(tuple(x.shape), ctx.dtype)
        ops.scale_add_rmsnorm(x, alpha, delta, self.w["weight"], self.eps, copy)
        return x if copy is None else copy
