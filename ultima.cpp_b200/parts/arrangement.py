"""How a layer's parts are arranged around the residual stream."""
from __future__ import annotations

from .base import Arrangement, register_part


@register_part("arrangement", "pre_norm")
class PreNorm(Arrangement):
    """x += mixer(norm(x)); x += feed_forward(norm(x)), the residual stream x in float32
    (reference: src/model/qwen_block.cpp:621-628, :782-792, :811-812)."""

    roles = {"mixer_norm": "norm", "mixer": "mixer", "feed_forward_norm": "norm",
             "feed_forward": "feed_forward"}

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
