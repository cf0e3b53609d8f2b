"""RMSNorm as a part. Formula and rounding: src/gpu/cuda/shaders/rms_norm.cu:78-115 of the
reference (sum of squares and scaling in float, weight used as stored)."""
from __future__ import annotations

from .base import Param, Part, Source, register_part


class RMSNorm(Part):
    graph_safe = True

    def __init__(self, size: int, eps: float, weight_name: str = "weight"):
        self.size, self.eps, self.weight_name = size, float(eps), weight_name
        self.weight = None

    def params(self):
        return [Param("weight", (Source(self.weight_name, (self.size,), init="norm"),), role="vector")]

    def forward(self, h, ctx):
        """h: float32 residual stream [T, size] -> normalised activations in the run dtype."""
        return ctx.backend.rmsnorm(h, self.weight, self.eps)

    def deferred(self, h, ctx, rows=None):
        """The same norm (of rows `rows` of h when given) for a consumer that may run it inside its
        own first product: a tensor, or the backend's deferred form that its products accept."""
        return ctx.backend.normed(h, self.weight, self.eps, rows)

    def forward_f32(self, h, ctx):
        import torch
        return ctx.backend.rmsnorm(h, self.weight, self.eps, out_dtype=torch.float32)


register_part("norm", "rmsnorm", RMSNorm)
