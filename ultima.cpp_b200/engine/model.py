"""A model built from its description: parts made, weights bound, and the forward pass of
one step over the run list."""
from __future__ import annotations

import os
import sys

import torch

# ULTIMA_TRACE=1: a line for every run of a layer with the sum of the residual stream behind it, in
# the form of the reference's trace ("name-layer = {n} sum = ...", src/model/qwen_block.cpp:29-42),
# so that two runs (32-bit and bfloat16, or two ways of cutting a prompt) can be compared line by line.
TRACE = os.environ.get("ULTIMA_TRACE", "") not in ("", "0")


def _trace(name: str, index: int, x: torch.Tensor) -> None:
    print(f"{name}-{index} = {{{x.numel()}}} sum = {x.double().sum().item():.6f}", file=sys.stderr, flush=True)

from ..parts.base import ModelSpec, build_part


class BuiltLayer:
    """A layer's arrangement and its parts, built and bound; a part is reached by its role
    (``layer.mixer``, ``layer.parts["mixer"]``)."""

    def __init__(self, arrangement, parts: dict):
        self.arrangement, self.parts = arrangement, dict(parts)
        for role, p in parts.items():
            setattr(self, role, p)
        holders = [p for p in parts.values() if getattr(p, "cache_need", None) is not None and p.cache_need() is not None]
        if len(holders) > 1:
            raise ValueError("a layer may hold one part that keeps a cache; this one has "
                             + ", ".join(f"{p.family} '{p.kind}'" for p in holders))
        self.cache_holder = holders[0] if holders else None

    def cache_need(self):
        return self.cache_holder.cache_need() if self.cache_holder is not None else None

    @property
    def graph_safe(self) -> bool:
        return all(getattr(p, "graph_safe", False) for p in self.parts.values())


class Model:
    def __init__(self, spec: ModelSpec, tensors: dict, rt):
        """tensors: full tensor name -> tensor on the runtime's device, already in their
        storage types."""
        self.spec, self.rt = spec, rt

        def bound(family, ps, prefix):
            p = build_part(family, ps)
            p.bind({s.name: tensors[prefix + s.name] for s in p.weight_specs()}, rt)
            return p

        self.embedding = bound("embedding", spec.embedding, spec.embedding_name)
        self.layers = []
        for L in spec.layers:
            arrangement = build_part("arrangement", L.arrangement)
            parts = {role: bound(family, L.part(role), L.name_of(role)) for role, family in L.roles().items()}
            self.layers.append(BuiltLayer(arrangement, parts))
        self.final_norm = bound("norm", spec.final_norm, spec.final_norm_name)
        self.head = build_part("head", spec.head)
        if spec.head.get("tied"):
            self.head.bind({"weight": self.embedding.table}, rt)
        else:
            self.head.bind({s.name: tensors[spec.head_name + s.name] for s in self.head.weight_specs()}, rt)
        for r in spec.runs:
            if not (0 <= r.layer < len(self.layers)):
                raise ValueError(f"run list names layer {r.layer}; the model has {len(self.layers)}")
        self._stack = None            # see _stack_plan

    def all_parts(self) -> list:
        return [self.embedding, self.final_norm, self.head] + [p for L in self.layers for p in L.parts.values()]

    def cache_needs(self):
        """For each run of the run list, what its layer asks of the cache."""
        return [self.layers[r.layer].cache_need() for r in self.spec.runs]

    def cache_sources(self):
        return [r.cache_from for r in self.spec.runs]

    def _stack_plan(self, cache):
        """The plan that runs all layers of a decode step as one resident kernel, if this model's layers
        are of the kinds that kernel takes (kernels/decode_stack.py); None otherwise."""
        if self._stack is None:
            from ..kernels import decode_stack
            self._stack = decode_stack.StackPlan(self, self.rt, cache) if not TRACE and \
                decode_stack.StackPlan.fits(self, self.rt, cache) else False
        return self._stack or None

    def forward(self, batch, cache) -> torch.Tensor:
        """Logits (float32 [wanted rows, vocabulary]) of one step; the cache is read and
        extended in place."""
        rt = self.rt
        rt.arena.reset(0)
        x = self.embedding.forward(batch.tok_ids, rt)
        if TRACE:
            _trace("embd", 0, x)
        plan = self._stack_plan(cache) if (batch.max_new == 1 and batch.n_tokens <= 64) else None
        if plan is not None:
            plan.run(x, batch)                    # one token a sequence: the whole stack in one kernel
        else:
            for i, r in enumerate(self.spec.runs):
                layer = self.layers[r.layer]
                layer.arrangement.run(layer, x, batch, cache.run_cache(i, batch.tables), rt)
                if TRACE:
                    _trace("l_out", i, x)
        if batch.want_rows.numel() == 0:
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=rt.device)
        h = self.final_norm.forward(x, rt, rows=batch.want_rows)
        return self.head.forward(h, rt)
