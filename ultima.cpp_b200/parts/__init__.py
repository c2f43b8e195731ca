"""Parts a layer is put together from, and the description of a model as data."""
from .base import (PartSpec, part, register_part, part_class, build_part, Part, Norm, Position,
                   Mixer, FeedForward, KVNeed, StateNeed, LayerSpec, Run, ModelSpec, FAMILIES)
from . import norm, position, attention, mlp, arrangement, embedding   # registers the parts

__all__ = ["PartSpec", "part", "register_part", "part_class", "build_part", "Part", "Norm",
           "Position", "Mixer", "FeedForward", "KVNeed", "StateNeed", "LayerSpec", "Run",
           "ModelSpec", "FAMILIES"]
