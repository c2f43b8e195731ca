"""Parts of a layer, the tables they are registered in, and the data that describes a model.

A model is data: a list of layers, each naming its mixer, feed-forward, norms and how they
are arranged, plus a run list that says in which order layers run and whose cache each run
uses.  Every part takes its sizes and constants as parameters and is looked up by name in
a table, so a part defined elsewhere (a test, another package) can be registered and used
without touching these files.  No part knows which model it is in.

The reference makes the same choices with flags inside one block function (FFN kind,
activation, QKV kind and rotary style per architecture, include/ultima/model/arch_registry.hpp:
43-67; per-layer flag vectors such as ``layer_is_swa``, include/ultima/model/imodel.hpp:63-69).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

from ..weights.spec import WeightSpec


@dataclass(frozen=True)
class PartSpec:
    """Which part (``kind`` is a key of the family's table) and its parameters."""
    kind: str
    params: tuple = ()                       # sorted (key, value) pairs; see ``part()``

    def get(self, key, default=None):
        return dict(self.params).get(key, default)

    def as_dict(self) -> dict:
        return dict(self.params)


def part(kind: str, **params) -> PartSpec:
    return PartSpec(kind, tuple(sorted(params.items())))


FAMILIES = ("norm", "position", "mixer", "feed_forward", "arrangement", "embedding", "head")
_TABLES: dict[str, dict[str, type]] = {f: {} for f in FAMILIES}


def register_part(family: str, kind: str, replace: bool = False):
    """Class decorator: ``@register_part("mixer", "my_mixer")``."""
    if family not in _TABLES:
        raise KeyError(f"unknown part family '{family}' (families: {', '.join(FAMILIES)})")

    def deco(cls):
        if kind in _TABLES[family] and not replace and _TABLES[family][kind] is not cls:
            raise KeyError(f"{family} '{kind}' is already registered")
        _TABLES[family][kind] = cls
        cls.family, cls.kind = family, kind
        return cls
    return deco


def part_class(family: str, kind: str) -> type:
    try:
        return _TABLES[family][kind]
    except KeyError:
        known = ", ".join(sorted(_TABLES.get(family, {})))
        raise KeyError(f"no {family} named '{kind}' is registered (known: {known})") from None


def build_part(family: str, spec: PartSpec):
    return part_class(family, spec.kind)(**spec.as_dict())


# ---------------------------------------------------------------------------------------
# what a mixer asks of the cache
# ---------------------------------------------------------------------------------------
@dataclass(frozen=True)
class KVNeed:
    """Keys and values for every position (``window`` None) or for the last ``window``."""
    n_kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class StateNeed:
    """Per-sequence state of fixed size: ``shape`` elements of ``dtype`` ("float32"...), zero at
    a sequence's start."""
    shape: tuple
    dtype: str = "float32"


class Part:
    """Base of every part.  Weight names are relative to the part ("q_proj.weight")."""
    family = ""
    kind = ""

    def weight_specs(self) -> list[WeightSpec]:
        return []

    def bind(self, tensors: dict, rt) -> None:
        """Take the loaded tensors (relative names) and prepare for running on ``rt``."""

    def scratch_bytes(self, n_tokens: int, rt) -> int:
        return 0


class Norm(Part):
    def forward(self, x, rt, rows=None):
        """x: float32 [T, width] -> activation-dtype [T or len(rows), width]."""
        raise NotImplementedError


class Position(Part):
    pass


class Mixer(Part):
    def cache_need(self):
        """None, a KVNeed, a StateNeed, or a tuple of both."""
        return None

    def forward(self, h, residual, batch, cache, rt) -> None:
        """h: normed activations [T, width]; add the mixer's output into ``residual``
        (float32 [T, width]).  ``cache`` is this run's view of the cache (or None)."""
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, h, residual, batch, rt) -> None:
        raise NotImplementedError


# ---------------------------------------------------------------------------------------
# the description of a model
# ---------------------------------------------------------------------------------------
@dataclass(frozen=True)
class LayerSpec:
    arrangement: PartSpec
    mixer: PartSpec
    feed_forward: PartSpec
    mixer_norm: PartSpec
    feed_forward_norm: PartSpec
    prefix: str = ""                                        # "model.layers.3."
    names: tuple = (("mixer", "mixer."), ("feed_forward", "feed_forward."),
                    ("mixer_norm", "mixer_norm."), ("feed_forward_norm", "feed_forward_norm."))

    def name_of(self, role: str) -> str:
        return self.prefix + dict(self.names)[role]


@dataclass(frozen=True)
class Run:
    """One entry of the run list: run ``layer``; ``cache_from`` names an earlier entry (by its
    index in the run list) whose cache this run reads instead of keeping its own."""
    layer: int
    cache_from: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    width: int
    vocab_size: int
    max_positions: int
    embedding: PartSpec
    embedding_name: str
    layers: tuple
    runs: tuple
    final_norm: PartSpec
    final_norm_name: str
    head: PartSpec
    head_name: str
    stop_token_ids: tuple = ()

    def parts_with_names(self):
        """(name prefix, family, PartSpec) for every part that owns weights."""
        out = [(self.embedding_name, "embedding", self.embedding)]
        for L in self.layers:
            out.append((L.name_of("mixer_norm"), "norm", L.mixer_norm))
            out.append((L.name_of("mixer"), "mixer", L.mixer))
            out.append((L.name_of("feed_forward_norm"), "norm", L.feed_forward_norm))
            out.append((L.name_of("feed_forward"), "feed_forward", L.feed_forward))
        out.append((self.final_norm_name, "norm", self.final_norm))
        out.append((self.head_name, "head", self.head))
        return out

    def weight_specs(self) -> list[WeightSpec]:
        specs, seen = [], set()
        for prefix, family, ps in self.parts_with_names():
            for s in build_part(family, ps).weight_specs():
                name = prefix + s.name
                if name in seen:
                    continue
                seen.add(name)
                specs.append(WeightSpec(name, s.shape, s.kind, s.init))
        return specs
