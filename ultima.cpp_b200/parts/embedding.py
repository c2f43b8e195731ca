"""Token embedding and the output head."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.spec import WeightSpec
from .base import Part, register_part


@register_part("embedding", "token_table")
class TokenTable(Part):
    """x_t = E[id_t, :], no scaling (reference: src/model/qwen_model.cpp:145-157).  A token id
    outside the vocabulary is refused on the host before the launch; the kernel checks again
    and raises a flag."""

    def __init__(self, vocab_size: int, width: int):
        self.vocab_size, self.width = int(vocab_size), int(width)
        self.table = None

    def weight_specs(self):
        return [WeightSpec("weight", (self.vocab_size, self.width))]

    def bind(self, tensors, rt):
        self.table = tensors["weight"].contiguous()
        self.status = rt.status[0:1]

    def forward(self, ids, rt):
        x = rt.arena.alloc((ids.numel(), self.width), torch.float32)
        rt.launches += 1
        ops.embed(self.table, ids, x, self.status)
        return x


@register_part("head", "linear")
class LinearHead(Part):
    """logits = W h, float32 out, no bias; ``tied`` takes the embedding table as W
    (reference: src/model/qwen_model.cpp:189-202, src/model/qwen_tensor_slots.cpp:150-158)."""

    def __init__(self, vocab_size: int, width: int, tied: bool):
        self.vocab_size, self.width, self.tied = int(vocab_size), int(width), bool(tied)
        self.weight = None

    def weight_specs(self):
        return [] if self.tied else [WeightSpec("weight", (self.vocab_size, self.width))]

    def bind(self, tensors, rt):
        self.weight = tensors["weight"].contiguous()

    def forward(self, h, rt):
        logits = torch.empty((h.shape[0], self.vocab_size), dtype=torch.float32, device=rt.device)
        rt.matmul(h, self.weight, logits)
        return logits
