"""Position encodings.  A mixer that rotates its queries and keys holds one of these."""
from __future__ import annotations

import torch

from .base import Position, register_part


@register_part("position", "rotary_half_split")
class RotaryHalfSplit(Position):
    """Rotation of the pairs (x[j], x[j + d/2]) by the angle pos * theta^(-2j/d)
    (reference: src/kernels/rope.cpp:17-52; the pairing is per-architecture data there,
    include/ultima/model/arch_registry.hpp:32-38).  The angles are formed in float64 on the
    host and the cosines and sines are stored as float32 tables [positions, d/2]; the
    rotation itself is float32 arithmetic in the kernel."""

    def __init__(self, head_dim: int, theta: float, max_positions: int):
        self.head_dim, self.theta, self.max_positions = int(head_dim), float(theta), int(max_positions)
        if self.head_dim % 2:
            raise ValueError("rotary head size must be even")
        self.cos = self.sin = None

    def bind(self, tensors, rt):
        key = ("rotary_half_split", self.head_dim, self.theta, self.max_positions)

        def make():
            half = self.head_dim // 2
            j = torch.arange(half, dtype=torch.float64)
            inv = 1.0 / torch.pow(torch.tensor(self.theta, dtype=torch.float64), 2.0 * j / self.head_dim)
            ang = torch.arange(self.max_positions, dtype=torch.float64)[:, None] * inv[None, :]
            return (torch.cos(ang).float().contiguous().to(rt.device),
                    torch.sin(ang).float().contiguous().to(rt.device))
        self.cos, self.sin = rt.shared(key, make)
