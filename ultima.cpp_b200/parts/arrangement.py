"""How a layer's parts are arranged around the residual stream."""
from __future__ import annotations

from .base import Part, register_part


@register_part("arrangement", "pre_norm")
class PreNorm(Part):
    """x += mixer(norm(x)); x += feed_forward(norm(x)), the residual stream x in float32
    (reference: src/model/qwen_block.cpp:621-628, :782-792, :811-812)."""

    def __init__(self):
        pass

    def run(self, layer, x, batch, cache, rt):
        mark = rt.arena.mark()
        h = layer.mixer_norm.forward(x, rt)
        layer.mixer.forward(h, x, batch, cache, rt)
        rt.arena.reset(mark)
        h = layer.feed_forward_norm.forward(x, rt)
        layer.feed_forward.forward(h, x, batch, rt)
        rt.arena.reset(mark)
