"""Feed-forward parts."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.spec import WeightSpec
from .base import FeedForward, register_part


@register_part("feed_forward", "gated_silu")
class GatedSiLU(FeedForward):
    """down(silu(gate(h)) * up(h)), no biases, added to the residual stream
    (reference: src/model/qwen_block.cpp:165-182, src/kernels/elementwise.cpp:62-68).
    Gate and up are held as one matrix [gate ; up]; the gate product is formed in float32
    from the float32 accumulators and rounded once."""

    graph_safe = True        # launches kernels only; no host work that depends on the data


    def __init__(self, width: int, inner: int):
        self.width, self.inner = int(width), int(inner)
        self.wgu = self.wd = None

    def weight_specs(self):
        return [WeightSpec("gate_proj.weight", (self.inner, self.width)),
                WeightSpec("up_proj.weight", (self.inner, self.width)),
                WeightSpec("down_proj.weight", (self.width, self.inner))]

    def bind(self, tensors, rt):
        g, u = tensors["gate_proj.weight"], tensors["up_proj.weight"]
        if g.dtype != u.dtype:
            raise ValueError("gate and up projections must share one element type")
        self.wd = tensors["down_proj.weight"].contiguous()
        # On the tensor-core path blocks of 64 gate rows and 64 up rows alternate, so that one
        # 128-row tile of the product holds both halves of 64 features (see gemm_tcgen05.cu).
        self.interleaved = (rt.use_tensor_cores and g.dtype == torch.bfloat16 and self.inner % 64 == 0
                            and self.width % 8 == 0)
        if self.interleaved:
            n = self.inner // 64
            self.wgu = torch.stack([g.view(n, 64, self.width), u.view(n, 64, self.width)], dim=1) \
                .reshape(2 * self.inner, self.width).contiguous()
        else:
            self.wgu = torch.cat([g, u], dim=0).contiguous()

    def forward(self, h, residual, batch, rt):
        T = h.shape[0]
        a = rt.arena.alloc((T, self.inner), rt.dtype)
        if self.interleaved:
            rt.matmul(h, self.wgu, a, ops.EPI_SWIGLU_IL)
        else:
            rt.matmul(h, self.wgu[:self.inner], a, ops.EPI_SWIGLU, w2=self.wgu[self.inner:])
        rt.matmul(a, self.wd, residual, ops.EPI_ADD)
