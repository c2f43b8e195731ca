"""Loading a model folder: every tensor a model asks for, by name, checked, then uploaded.

The reference resolves each weight by name with its expected shape and reports a missing
tensor or a shape mismatch (src/model/qwen_tensor_slots.cpp:23-64); here all faults of a
file are gathered and raised as one error.
"""
from __future__ import annotations

import json
import os

import torch

from .safetensors_io import open_safetensors
from .spec import WeightError, WeightSpec

_FLOATS = ("F64", "F32", "F16", "BF16")
_INTS = ("I64", "I32", "I16", "I8", "U8", "BOOL")


def storage_dtype(file_dtype: str, run_dtype: torch.dtype, kind: str) -> torch.dtype:
    """The type a tensor is held in on the device.

    32-bit run: every floating tensor in float32.  bfloat16 run: 16-bit matrices stay
    bfloat16 (float16 is converted), a tensor stored in 32-bit stays 32-bit, small vectors
    are widened to float32 (exact), integer tables are int32.
    """
    if file_dtype in _INTS or kind == "table":
        return torch.int32
    if run_dtype == torch.float32:
        return torch.float32
    if kind == "vector" or file_dtype in ("F32", "F64"):
        return torch.float32
    return torch.bfloat16


def _shard_files(model_dir: str) -> list[str]:
    index = os.path.join(model_dir, "model.safetensors.index.json")
    single = os.path.join(model_dir, "model.safetensors")
    if os.path.isfile(single):
        return [single]
    if os.path.isfile(index):
        with open(index, "r", encoding="utf-8") as f:
            wm = json.load(f).get("weight_map", {})
        return [os.path.join(model_dir, n) for n in sorted(set(wm.values()))]
    raise WeightError(f"no model.safetensors (or model.safetensors.index.json) in '{model_dir}'")


def _fit_error(model_dir, want: dict, where: dict, info, optional: tuple):
    """The one WeightError that lists everything that does not fit, or None."""
    missing = [n for n in want if n not in where]
    unexpected = sorted(n for n in where if n not in want and n not in optional)
    wrong_shape, wrong_dtype = [], []
    for n, s in want.items():
        if n not in where:
            continue
        dt, shape = info(n)
        if tuple(shape) != tuple(s.shape):
            wrong_shape.append((n, tuple(s.shape), tuple(shape)))
        if (s.kind == "table") != (dt in _INTS):
            wrong_dtype.append((n, "integer" if s.kind == "table" else "floating", dt))
    if not (missing or unexpected or wrong_shape or wrong_dtype):
        return None
    lines = [f"weights in '{model_dir}' do not fit the model:"]
    if missing:
        lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(missing))
    if unexpected:
        lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
    for n, exp, got in wrong_shape:
        lines.append(f"  wrong shape: '{n}' expected {list(exp)}, got {list(got)}")
    for n, exp, got in wrong_dtype:
        lines.append(f"  wrong dtype: '{n}' expected a {exp} type, got {got}")
    return WeightError("\n".join(lines), missing, unexpected, wrong_shape, wrong_dtype)


def check_weights(model_dir: str, specs: list[WeightSpec], optional: tuple = ()) -> dict:
    """Reads the headers only and raises the same WeightError as ``load_weights`` would; returns
    name -> (file dtype name, shape) of the model's tensors when everything fits."""
    from .safetensors_io import read_safetensors_header
    found = {}
    for path in _shard_files(model_dir):
        header, _, _ = read_safetensors_header(path)
        for n, e in header.items():
            found[n] = (e["dtype"], tuple(int(x) for x in e["shape"]))
    want = {s.name: s for s in specs}
    err = _fit_error(model_dir, want, found, lambda n: found[n], optional)
    if err is not None:
        raise err
    return {n: found[n] for n in want}


def load_weights(model_dir: str, specs: list[WeightSpec], run_dtype: torch.dtype,
                 device: str | torch.device = "cpu", optional: tuple = ()) -> dict:
    """name -> tensor on ``device``.  ``optional`` names may be present and are then ignored
    (a tied head that a file stores all the same)."""
    files = [open_safetensors(p) for p in _shard_files(model_dir)]
    try:
        where = {}
        for f in files:
            for n in f.names():
                where[n] = f
        want = {s.name: s for s in specs}
        err = _fit_error(model_dir, want, where, lambda n: where[n].info(n), optional)
        if err is not None:
            raise err
        out = {}
        for n, s in want.items():
            dt, _ = where[n].info(n)
            t = where[n].tensor(n)
            out[n] = t.to(device=device, dtype=storage_dtype(dt, run_dtype, s.kind)).contiguous()
        return out
    finally:
        for f in files:
            f.close()
