"""Parts a layer is put together from, and the description of a model as data."""
from .base import (PartSpec, part, register_part, part_class, build_part, Part, Norm, Position, Rotation,
                   Mixer, FeedForward, Arrangement, KVNeed, StateNeed, LayerSpec, layer, Run, ModelSpec, FAMILIES)
from . import norm, position, attention, mlp, arrangement, embedding   # registers the parts

__all__ = ["PartSpec", "part", "register_part", "part_class", "build_part", "Part", "Norm",
           "Position", "Rotation", "Mixer", "FeedForward", "Arrangement", "KVNeed", "StateNeed",
           "LayerSpec", "layer", "Run", "ModelSpec", "FAMILIES"]
