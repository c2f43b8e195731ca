"""Random weights from a seed, and the model folder that holds them.

Each tensor has its own key, made from the seed and the tensor's name, and element ``i`` of
the tensor is a function of (key, i) only: a counter-based generator.  It is written three
times with the same bits: here in numpy (``counter_normal``), in CUDA (``ub_fill_normal`` in
csrc/basic.cu, for models too large to draw on the host) and, as the tests' own copy, in
tests/plain_random.py; so a model drawn on the device can be drawn again on the host, value
for value.  Distributions: projections and the embedding N(0, std), norm weights 1 + N(0, std);
the std comes with the weight spec.

How a draw is made (every step an integer operation or one correctly rounded float32
operation, so that the three implementations agree bit for bit):
    r  = mix64(key ^ mix64(i))                     SplitMix64's finaliser
    u1 = ((r >> 41) + 0.5) * 2^-23                 in (0, 1)
    t  = (r >> 16) & 0xFFFFFF                       the angle 2 pi t / 2^24
    z  = sqrt(-2 ln u1) * cos(2 pi t / 2^24)       Box-Muller, with a logarithm and a cosine made
                                                   of float32 additions and multiplications
"""
from __future__ import annotations

import hashlib
import json
import os

import numpy as np
import torch

from .safetensors_io import write_safetensors
from .spec import WeightSpec

_M64 = np.uint64(0xFFFFFFFFFFFFFFFF)


def _mix64(z: np.ndarray) -> np.ndarray:
    z = z + np.uint64(0x9E3779B97F4A7C15)
    z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
    z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
    return z ^ (z >> np.uint64(31))


def _f(bits: int) -> np.float32:
    return np.array([bits], dtype=np.uint32).view(np.float32)[0]


def counter_normal(key: int, start: int, count: int) -> np.ndarray:
    """Standard normal draws of the elements start .. start + count - 1 under ``key`` (float32)."""
    f32, u32 = np.float32, np.uint32
    with np.errstate(over="ignore"):
        i = np.arange(start, start + count, dtype=np.uint64)
        r = _mix64(np.uint64(key & 0xFFFFFFFFFFFFFFFF) ^ _mix64(i))
    # ln(u1)
    u1 = ((r >> np.uint64(41)).astype(f32) + f32(0.5)) * _f(0x34000000)
    ub = u1.view(u32)
    e = (ub >> u32(23)).astype(np.int32) - np.int32(127)
    m = ((ub & u32(0x7FFFFF)) | u32(0x3F800000)).view(f32)
    big = m > _f(0x3FB504F3)
    m = np.where(big, m * f32(0.5), m)
    e = e + big.astype(np.int32)
    s = (m - f32(1.0)) / (m + f32(1.0))
    s2 = s * s
    p = np.full(count, _f(0x3DBA2E8C), dtype=f32)
    for c in (0x3DE38E39, 0x3E124925, 0x3E4CCCCD, 0x3EAAAAAB):
        p = p * s2 + _f(c)
    p = p * s2 + f32(1.0)
    ln_m = (f32(2.0) * s) * p
    ln_u = e.astype(f32) * _f(0x3F317218) + ln_m
    rad = np.sqrt(f32(-2.0) * ln_u)
    # cos(2 pi t / 2^24)
    t = ((r >> np.uint64(16)) & np.uint64(0xFFFFFF)).astype(u32)
    quad, rest = t >> u32(22), t & u32(0x3FFFFF)
    fold = rest > u32(0x200000)
    fr = np.where(fold, u32(0x400000) - rest, rest)
    x = (fr.astype(f32) * _f(0x34800000)) * _f(0x3FC90FDB)
    x2 = x * x
    sn = np.full(count, _f(0x3638EF1D), dtype=f32)
    for c in (0x39500D01, 0x3C088889, 0x3E2AAAAB):
        sn = _f(c) - sn * x2
    sn = (f32(1.0) - sn * x2) * x
    cs = np.full(count, _f(0x3493F27E), dtype=f32)
    for c in (0x37D00D01, 0x3AB60B61, 0x3D2AAAAB):
        cs = _f(c) - cs * x2
    cs = f32(0.5) - cs * x2
    cs = f32(1.0) - cs * x2
    sin_q, cos_q = np.where(fold, cs, sn), np.where(fold, sn, cs)
    c = np.where(quad == 0, cos_q, np.where(quad == 1, -sin_q, np.where(quad == 2, -cos_q, sin_q)))
    return (rad * c).astype(f32, copy=False)


def counter_fill(shape, key: int, shift: float, std: float, chunk: int = 1 << 16) -> torch.Tensor:
    """float32 tensor of ``shape``: shift + std * counter_normal(key, i), i the flat index."""
    n = 1
    for d in shape:
        n *= int(d)
    out = np.empty(n, dtype=np.float32)
    sh, sd = np.float32(shift), np.float32(std)
    for a in range(0, n, chunk):
        b = min(n, a + chunk)
        out[a:b] = sh + sd * counter_normal(key, a, b - a)
    return torch.from_numpy(out).view(*shape)


def _tensor_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode("utf-8")).digest()
    return int.from_bytes(h[:8], "little") & ((1 << 63) - 1)


def random_tensors(specs: list[WeightSpec], seed: int, dtype: torch.dtype = torch.float32) -> dict:
    """name -> CPU tensor.  Floating tensors are drawn in float32 and then rounded to ``dtype``."""
    out = {}
    for s in specs:
        if s.kind == "table":
            out[s.name] = torch.zeros(s.shape, dtype=torch.int32)
            continue
        if s.init[0] == "zeros":
            t = torch.zeros(s.shape, dtype=torch.float32)
        elif s.init[0] in ("normal", "one_plus_normal"):
            t = counter_fill(s.shape, _tensor_seed(seed, s.name), 1.0 if s.init[0] == "one_plus_normal" else 0.0,
                             float(s.init[1]))
        else:
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
    host in reasonable time): the values of ``random_tensors`` for the same seed, bit for bit, in
    the storage types the loader would give them."""
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
