"""Position encodings.  A mixer that encodes its queries and keys by position holds one of these."""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import Position, Rotation, register_part


class _Rotary(Position):
    """Rotation of pairs of a head's first ``rotary_dim`` columns by the angle pos * theta^(-2j/rotary_dim)
    for pair j; the other columns pass through (reference: src/kernels/rope.cpp:17-52; ``rope_dim``
    smaller than the head :27, :50).  Which two columns make pair j is the subclass's: the pairing is
    per-architecture data in the reference (include/ultima/model/arch_registry.hpp:32-38).  The angles
    are formed in float64 on the host and the cosines and sines are stored as float32 tables
    [positions, rotary_dim / 2]; the rotation itself is float32 arithmetic in the kernels."""

    interleaved = False
    graph_safe = True        # tables made at bind; forward launches kernels only

    def __init__(self, head_dim: int, theta: float, max_positions: int, rotary_dim: int | None = None):
        self.head_dim, self.theta, self.max_positions = int(head_dim), float(theta), int(max_positions)
        self.rotary_dim = int(rotary_dim) if rotary_dim is not None else self.head_dim
        if self.rotary_dim % 2 or not (2 <= self.rotary_dim <= self.head_dim):
            raise ValueError(f"rotary size {self.rotary_dim} must be even and at most the head size {self.head_dim}")
        self.cos = self.sin = None

    def bind(self, tensors, rt):
        key = ("rotary", self.rotary_dim, self.theta, self.max_positions)

        def make():
            half = self.rotary_dim // 2
            j = torch.arange(half, dtype=torch.float64)
            inv = 1.0 / torch.pow(torch.tensor(self.theta, dtype=torch.float64), 2.0 * j / self.rotary_dim)
            ang = torch.arange(self.max_positions, dtype=torch.float64)[:, None] * inv[None, :]
            return (torch.cos(ang).float().contiguous().to(rt.device),
                    torch.sin(ang).float().contiguous().to(rt.device))
        self.cos, self.sin = rt.shared(key, make)

    def rotation(self):
        return Rotation(self.cos, self.sin, self.rotary_dim, self.interleaved)

    def forward(self, q, k, positions, rt):
        for x in (q, k):
            rt.launches += 1
            ops.rotate_pairs(x, self.cos, self.sin, positions, self.rotary_dim, self.interleaved)


@register_part("position", "rotary_half_split")
class RotaryHalfSplit(_Rotary):
    """Pair j is (x[j], x[j + rotary_dim / 2]) (src/kernels/rope.cpp:42-43)."""
    interleaved = False


@register_part("position", "rotary_interleaved")
class RotaryInterleaved(_Rotary):
    """Pair j is (x[2j], x[2j + 1])."""
    interleaved = True
