"""Choosing the next token: parameters and the sampler that runs the kernel."""
from .params import SamplingParams
from .sampler import Sampler, uniform_of

__all__ = ["SamplingParams", "Sampler", "uniform_of"]
