"""ultima_b200: a small model library with generation of its own for one NVIDIA B200.

Everything between a request's token ids and its next token, for the Qwen3 dense
architecture of tattooinmtl/Ultima.cpp: configuration and registry, safetensors weights,
layers put together from parts, a paged cache with slots, one step function, a generation
loop, sampling, trace replay, and hand-written CUDA kernels for sm_100a.
"""
from . import config, weights, parts, cache, arch
from .config import ConfigError, Qwen3Config, config_from_dir, config_from_dict
from .weights import WeightError, write_random_model
from .arch import model_spec_for

__version__ = "0.1.0"


def __getattr__(name):
    # the engine pulls in torch.cuda and the kernels; load it on first use
    import importlib
    if name in ("engine", "sampling", "kernels", "cli"):
        return importlib.import_module(f"{__name__}.{name}")
    if name in ("Engine", "StepError"):
        return getattr(importlib.import_module(f"{__name__}.engine"), name)
    if name in ("LLM", "Generation", "generate", "load"):
        return getattr(importlib.import_module(f"{__name__}.engine.generate"), name)
    if name in ("SamplingParams", "Sampler"):
        return getattr(importlib.import_module(f"{__name__}.sampling"), name)
    raise AttributeError(f"module '{__name__}' has no attribute '{name}'")
