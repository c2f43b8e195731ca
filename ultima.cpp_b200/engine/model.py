"""A model built from its description: parts made, weights bound, and the forward pass of
one step over the run list."""
from __future__ import annotations

import os
import sys
from dataclasses import dataclass

import torch

# ULTIMA_TRACE=1: a line for every run of a layer with the sum of the residual stream behind it, in
# the form of the reference's trace ("name-layer = {n} sum = ...", src/model/qwen_block.cpp:29-42),
# so that two runs (32-bit and bfloat16, or two ways of cutting a prompt) can be compared line by line.
TRACE = os.environ.get("ULTIMA_TRACE", "") not in ("", "0")


def _trace(name: str, index: int, x: torch.Tensor) -> None:
    print(f"{name}-{index} = {{{x.numel()}}} sum = {x.double().sum().item():.6f}", file=sys.stderr, flush=True)

from ..parts.base import ModelSpec, build_part


@dataclass
class BuiltLayer:
    arrangement: object
    mixer: object
    feed_forward: object
    mixer_norm: object
    feed_forward_norm: object


class Model:
    def __init__(self, spec: ModelSpec, tensors: dict, rt):
        """tensors: full tensor name -> tensor on the runtime's device, already in their
        storage types."""
        self.spec, self.rt = spec, rt

        def bound(family, ps, prefix):
            p = build_part(family, ps)
            rel = {s.name: tensors[prefix + s.name] for s in p.weight_specs()}
            return p, rel

        self.embedding, rel = bound("embedding", spec.embedding, spec.embedding_name)
        self.embedding.bind(rel, rt)
        self.layers = []
        for L in spec.layers:
            parts = {}
            for role, family, ps in (("mixer_norm", "norm", L.mixer_norm), ("mixer", "mixer", L.mixer),
                                     ("feed_forward_norm", "norm", L.feed_forward_norm),
                                     ("feed_forward", "feed_forward", L.feed_forward)):
                p, rel = bound(family, ps, L.name_of(role))
                p.bind(rel, rt)
                parts[role] = p
            self.layers.append(BuiltLayer(arrangement=build_part("arrangement", L.arrangement), **parts))
        self.final_norm, rel = bound("norm", spec.final_norm, spec.final_norm_name)
        self.final_norm.bind(rel, rt)
        self.head, rel = bound("head", spec.head, spec.head_name)
        if spec.head.get("tied"):
            rel = {"weight": self.embedding.table}
        self.head.bind(rel, rt)
        for r in spec.runs:
            if not (0 <= r.layer < len(self.layers)):
                raise ValueError(f"run list names layer {r.layer}; the model has {len(self.layers)}")

    def cache_needs(self):
        """For each run of the run list, what its mixer asks of the cache."""
        return [self.layers[r.layer].mixer.cache_need() for r in self.spec.runs]

    def cache_sources(self):
        return [r.cache_from for r in self.spec.runs]

    def forward(self, batch, cache) -> torch.Tensor:
        """Logits (float32 [wanted rows, vocabulary]) of one step; the cache is read and
        extended in place."""
        rt = self.rt
        rt.arena.reset(0)
        x = self.embedding.forward(batch.tok_ids, rt)
        if TRACE:
            _trace("embd", 0, x)
        for i, r in enumerate(self.spec.runs):
            layer = self.layers[r.layer]
            layer.arrangement.run(layer, x, batch, cache.run_cache(i, batch.tables), rt)
            if TRACE:
                _trace("l_out", i, x)
        if batch.want_rows.numel() == 0:
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=rt.device)
        h = self.final_norm.forward(x, rt, rows=batch.want_rows)
        return self.head.forward(h, rt)
