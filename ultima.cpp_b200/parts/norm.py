"""Norms."""
from __future__ import annotations

from ..kernels import ops
from ..weights.spec import WeightSpec
from .base import Norm, register_part


@register_part("norm", "rms")
class RMSNorm(Norm):
    """y = x * w / sqrt(mean(x^2) + eps): the weight multiplies (no 1 + w), no bias
    (reference: src/kernels/rmsnorm.cpp:10-17).  Input is the float32 residual stream, sums
    are float32, the output has the activation type."""

    def __init__(self, width: int, eps: float):
        self.width, self.eps = int(width), float(eps)
        self.weight = None

    def weight_specs(self):
        return [WeightSpec("weight", (self.width,), "vector", ("one_plus_normal", 0.05))]

    def bind(self, tensors, rt):
        self.weight = tensors["weight"].float().contiguous()

    def forward(self, x, rt, rows=None):
        n = x.shape[0] if rows is None else rows.numel()
        out = rt.arena.alloc((n, self.width), rt.dtype)
        rt.launches += 1
        ops.rmsnorm(x, self.weight, out, self.eps, rows)
        return out
