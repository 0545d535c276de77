"""RMSNorm with float32 statistics.

y = round(round(x * (mean(x^2) + eps)^-1/2) * w); ``add`` first forms the rounded
sum with the residual stream and returns it as the new stream
(tinyvllm/layers.py:129-164; tinyvllm/kernels/pointwise.cu:153-211).
"""

from __future__ import annotations

from ..ops import kernels
from .base import BuildContext, ParamSpec, Part
from .registry import register_part


class RMSNorm(Part):
    # y = x * rsqrt(mean(x^2) + eps) * weight: a projection behind it may apply it in its own kernel
    folds_into_product = True

    def __init__(self, ctx: BuildContext, *, width: int, eps: float, name: str | None = None) -> None:
        self.width = width
        self.eps = float(eps)
        self.name = name if name is not None else f"{ctx.prefix}.weight"
        self.weight = None

    def param_specs(self):
        return [ParamSpec.single("weight", self.name, (self.width,), role="vector", init="around_one")]

    def forward(self, x):
        return kernels.rms_norm(x, self.weight, self.eps)

    def add(self, x, residual):
        """(norm(x + residual), x + residual)"""
        return kernels.rms_norm(x, self.weight, self.eps, residual=residual)

    def add_rows(self, x, residual, rows):
        """norm(x + residual) on the rows named by ``rows`` only."""
        return kernels.rms_norm(x, self.weight, self.eps, residual=residual, rows=rows)


register_part("norm", "rms_norm", RMSNorm)
