"""The hand-written CUDA kernels behind their Python entry points."""
from . import build, ops
from .ops import KernelError

__all__ = ["build", "ops", "KernelError"]
