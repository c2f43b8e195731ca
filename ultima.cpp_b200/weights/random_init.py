"""Random weights from a seed, and the model folder that holds them.

Each tensor has its own generator, keyed by the seed and the tensor's name, so a tensor's
values do not depend on which other tensors the model has.  Distributions: projections and
the embedding N(0, std), norm weights 1 + N(0, std); the std comes with the weight spec.
"""
from __future__ import annotations

import hashlib
import json
import os

import torch

from .safetensors_io import write_safetensors
from .spec import WeightSpec


def _tensor_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode("utf-8")).digest()
    return int.from_bytes(h[:8], "little") & ((1 << 63) - 1)


def random_tensors(specs: list[WeightSpec], seed: int, dtype: torch.dtype = torch.float32) -> dict:
    """name -> CPU tensor.  Floating tensors are drawn in float32 and then rounded to ``dtype``."""
    out = {}
    for s in specs:
        g = torch.Generator(device="cpu")
        g.manual_seed(_tensor_seed(seed, s.name))
        if s.kind == "table":
            out[s.name] = torch.zeros(s.shape, dtype=torch.int32)
            continue
        if s.init[0] == "zeros":
            t = torch.zeros(s.shape, dtype=torch.float32)
        else:
            t = torch.randn(s.shape, generator=g, dtype=torch.float32) * float(s.init[1])
            if s.init[0] == "one_plus_normal":
                t = t + 1.0
            elif s.init[0] != "normal":
                raise ValueError(f"unknown init {s.init!r} for '{s.name}'")
        out[s.name] = t.to(dtype)
    return out


def write_random_model(model_dir: str, config, seed: int, dtype: str | None = None) -> str:
    """Write ``config.json`` and ``model.safetensors`` for ``config`` with weights from ``seed``."""
    from ..arch import model_spec_for      # late: arch imports parts imports weights
    dtype = dtype or config.torch_dtype
    tdt = {"bfloat16": torch.bfloat16, "float32": torch.float32, "float16": torch.float16}[dtype]
    spec = model_spec_for(config)
    tensors = random_tensors(spec.weight_specs(), seed, tdt)
    os.makedirs(model_dir, exist_ok=True)
    cfg = config.to_dict()
    cfg["torch_dtype"] = dtype
    with open(os.path.join(model_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(cfg, f, indent=1)
    write_safetensors(os.path.join(model_dir, "model.safetensors"), tensors,
                      metadata={"format": "pt", "seed": seed})
    return model_dir


def random_tensors_on_device(specs: list[WeightSpec], seed: int, run_dtype: torch.dtype, device) -> dict:
    """name -> tensor drawn on the GPU by the fill kernel (for models too large to draw on the
    host in reasonable time).  Same distributions as ``random_tensors``, other values."""
    from ..kernels import ops
    from .loader import storage_dtype
    out = {}
    file_dtype = "BF16" if run_dtype == torch.bfloat16 else "F32"
    for s in specs:
        dt = storage_dtype(file_dtype, run_dtype, s.kind)
        if s.kind == "table":
            out[s.name] = torch.zeros(s.shape, dtype=torch.int32, device=device)
            continue
        t = torch.empty(s.shape, dtype=dt, device=device)
        if s.init[0] == "zeros":
            t.zero_()
        else:
            shift = 1.0 if s.init[0] == "one_plus_normal" else 0.0
            ops.fill_normal(t, _tensor_seed(seed, s.name), shift, float(s.init[1]))
        out[s.name] = t
    return out
