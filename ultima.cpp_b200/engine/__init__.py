"""The runtime: the step function, the generation loop above it, and trace replay."""
from .runtime import Runtime, Arena
from .batch import StepBatch, build_step_batch
from .model import Model
from .engine import Engine, StepError

__all__ = ["Runtime", "Arena", "StepBatch", "build_step_batch", "Model", "Engine", "StepError"]
