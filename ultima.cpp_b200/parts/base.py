"""Parts of a layer, the tables they are registered in, and the data that describes a model.

A model is data: a list of layers, each naming its arrangement and the part that plays each
role the arrangement has (for the pre-norm block: mixer, feed-forward and their two norms), plus
a run list that says in which order layers run and whose cache each run uses.  Every part takes its sizes and constants as parameters and is looked up by name in
a table, so a part defined elsewhere (a test, another package) can be registered and used
without touching these files.  No part knows which model it is in.

The reference makes the same choices with flags inside one block function (FFN kind,
activation, QKV kind and rotary style per architecture, include/ultima/model/arch_registry.hpp:
43-67; per-layer flag vectors such as ``layer_is_swa``, include/ultima/model/imodel.hpp:63-69).
"""
from __future__ import annotations

from dataclasses import dataclass
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
    # True: ``forward`` only launches kernels on tensors of the step's arena, the cache and the step
    # record, and does no host work that depends on their values, so a step that runs it can be
    # captured as a CUDA graph and replayed.  A part that reads results on the host leaves it False.
    graph_safe = False

    def weight_specs(self) -> list[WeightSpec]:
        return []

    def bind(self, tensors: dict, rt) -> None:
        """Take the loaded tensors (relative names) and prepare for running on ``rt``.  A part
        that cannot run with its sizes (a head size no kernel takes) says so here, with a
        ValueError, so that the fault shows when the engine is built and not in a step."""

    def scratch_bytes(self, n_tokens: int, rt) -> int:
        return 0

    def kernel_needs(self, run_dtype) -> list:
        """The libraries of csrc/ this part launches, as (source, (defines...)) pairs, beyond the
        ones every model uses; they are compiled together when the engine is built."""
        return []


class Norm(Part):
    graph_safe = True

    def forward(self, x, rt, rows=None):
        """x: float32 [T, width] -> activation-dtype [T or len(rows), width]."""
        raise NotImplementedError


@dataclass
class Rotation:
    """A position encoding in the form the fused kernels apply themselves: pairs of a head's
    first ``dim`` columns are rotated by angles that depend on the position, the other columns
    pass through.  cos, sin: float32 [positions, dim / 2] on the device.  ``interleaved``: the
    pairs are (2j, 2j + 1) instead of (j, j + dim / 2)."""
    cos: object
    sin: object
    dim: int
    interleaved: bool = False


class Position(Part):
    """A position encoding of queries and keys.  A mixer that holds one calls ``forward`` on the
    queries and keys of the step's tokens before the keys go into the cache.  An encoding that
    is a rotation of pairs may also describe itself with ``rotation()``; the attention part then
    hands the tables to kernels that rotate while they norm and write the cache, and never
    calls ``forward``.  Both must give the same result.  A mixer that holds a position encoding
    is graph_safe only if the encoding is."""

    def rotation(self) -> Optional[Rotation]:
        return None

    def forward(self, q, k, positions, rt) -> None:
        """Encode in place.  q: [T, heads, head size], k: [T, kv heads, head size] (views with a
        last stride of 1, element type of the activations), positions: int32 [T] absolute."""
        raise NotImplementedError


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


class Arrangement(Part):
    """How a layer's parts stand around the residual stream.  ``roles`` names the parts a layer
    of this arrangement has, role -> family; the model builds exactly those, from the layer's
    ``LayerSpec.parts``, and hands them to ``run`` as attributes of ``layer``.  At most one of
    them may ask for a cache (``cache_need``): it gets the run's view of the cache."""
    roles: dict = {}

    def run(self, layer, x, batch, cache, rt) -> None:
        """Update the residual stream x (float32 [T, width]) in place."""
        raise NotImplementedError


# ---------------------------------------------------------------------------------------
# the description of a model
# ---------------------------------------------------------------------------------------
@dataclass(frozen=True)
class LayerSpec:
    """One layer: its arrangement and, for each role the arrangement names, the part that
    plays it.  ``names`` gives a role's tensor-name prefix below ``prefix`` (default: the role
    and a dot), so that a layer can follow a checkpoint's own names."""
    arrangement: PartSpec
    parts: tuple = ()                                       # ((role, PartSpec), ...)
    prefix: str = ""                                        # "model.layers.3."
    names: tuple = ()                                       # ((role, "self_attn."), ...)

    def part(self, role: str) -> PartSpec:
        for r, ps in self.parts:
            if r == role:
                return ps
        raise KeyError(f"layer '{self.prefix}' has no part in the role '{role}' "
                       f"(it has: {', '.join(r for r, _ in self.parts)})")

    def name_of(self, role: str) -> str:
        return self.prefix + dict(self.names).get(role, role + ".")

    def roles(self) -> dict:
        """role -> family, as the layer's arrangement declares them."""
        return dict(part_class("arrangement", self.arrangement.kind).roles)


def layer(arrangement: PartSpec, prefix: str = "", names=(), **roles) -> LayerSpec:
    """``layer(part("pre_norm"), prefix="l0.", mixer=..., feed_forward=..., mixer_norm=..., ...)``"""
    want = part_class("arrangement", arrangement.kind).roles
    for r in want:
        if r not in roles:
            raise KeyError(f"arrangement '{arrangement.kind}' needs a part in the role '{r}'")
    for r in roles:
        if r not in want:
            raise KeyError(f"arrangement '{arrangement.kind}' has no role '{r}' (roles: {', '.join(want)})")
    return LayerSpec(arrangement, tuple((r, roles[r]) for r in want), prefix,
                     tuple(dict(names).items()) if not isinstance(names, tuple) else names)


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
            for role, family in L.roles().items():
                out.append((L.name_of(role), family, L.part(role)))
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

    def kernel_needs(self, run_dtype) -> list:
        """Every library the model's parts ask for (see ``Part.kernel_needs``), once each."""
        out = []
        for _, family, ps in self.parts_with_names():
            for t in build_part(family, ps).kernel_needs(run_dtype):
                t = (t[0], tuple(t[1]))
                if t not in out:
                    out.append(t)
        return out
