"""The safetensors container: an 8-byte little-endian header length, a JSON header that
maps each tensor name to its dtype, shape and byte range, then the raw little-endian data.

Reading goes through a memory map; nothing is copied until a tensor is asked for.
"""
from __future__ import annotations

import json
import mmap
import os
import struct

import numpy as np
import torch


class SafetensorsError(ValueError):
    pass


# safetensors dtype name -> (numpy dtype used to view the bytes, torch dtype, bytes per element)
_DTYPES = {
    "F64": (np.float64, torch.float64, 8), "F32": (np.float32, torch.float32, 4),
    "F16": (np.float16, torch.float16, 2), "BF16": (np.uint16, torch.bfloat16, 2),
    "I64": (np.int64, torch.int64, 8), "I32": (np.int32, torch.int32, 4),
    "I16": (np.int16, torch.int16, 2), "I8": (np.int8, torch.int8, 1),
    "U8": (np.uint8, torch.uint8, 1), "BOOL": (np.bool_, torch.bool, 1),
}
_TORCH_TO_NAME = {v[1]: k for k, v in _DTYPES.items()}


def read_safetensors_header(path: str):
    """(header dict without __metadata__, offset of the data section, file size)."""
    size = os.path.getsize(path)
    with open(path, "rb") as f:
        head = f.read(8)
        if len(head) < 8:
            raise SafetensorsError(f"{path}: file too short for a safetensors header")
        (n,) = struct.unpack("<Q", head)
        if n <= 0 or 8 + n > size:
            raise SafetensorsError(f"{path}: header length {n} does not fit the file ({size} bytes)")
        raw = f.read(n)
    try:
        header = json.loads(raw.decode("utf-8"))
    except (UnicodeDecodeError, json.JSONDecodeError) as e:
        raise SafetensorsError(f"{path}: header is not JSON: {e}") from e
    if not isinstance(header, dict):
        raise SafetensorsError(f"{path}: header must be a JSON object")
    header.pop("__metadata__", None)
    data_start = 8 + n
    data_len = size - data_start
    spans = []
    for name, info in header.items():
        try:
            dt, shape, (b, e) = info["dtype"], info["shape"], info["data_offsets"]
        except (KeyError, TypeError, ValueError) as err:
            raise SafetensorsError(f"{path}: bad header entry for '{name}'") from err
        if dt not in _DTYPES:
            raise SafetensorsError(f"{path}: tensor '{name}' has unsupported dtype {dt}")
        count = 1
        for s in shape:
            count *= int(s)
        if e - b != count * _DTYPES[dt][2]:
            raise SafetensorsError(f"{path}: tensor '{name}' byte range {b}:{e} does not match "
                                   f"shape {shape} of {dt}")
        if b < 0 or e > data_len:
            raise SafetensorsError(f"{path}: tensor '{name}' byte range {b}:{e} lies outside the "
                                   f"data section ({data_len} bytes); file truncated?")
        spans.append((b, e, name))
    spans.sort()
    for (b0, e0, n0), (b1, e1, n1) in zip(spans, spans[1:]):
        if b1 < e0:
            raise SafetensorsError(f"{path}: tensors '{n0}' and '{n1}' overlap")
    return header, data_start, size


class SafetensorsFile:
    """A memory-mapped safetensors file; ``tensor(name)`` gives a CPU torch tensor view."""

    def __init__(self, path: str):
        self.path = path
        self.header, self._start, self._size = read_safetensors_header(path)
        self._f = open(path, "rb")
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)

    def names(self):
        return list(self.header.keys())

    def info(self, name: str):
        e = self.header[name]
        return e["dtype"], tuple(int(s) for s in e["shape"])

    def tensor(self, name: str) -> torch.Tensor:
        e = self.header[name]
        np_dt, torch_dt, _ = _DTYPES[e["dtype"]]
        b, end = e["data_offsets"]
        shape = tuple(int(s) for s in e["shape"])
        count = int(np.prod(shape)) if shape else 1
        arr = np.frombuffer(self._mm, dtype=np_dt, count=count, offset=self._start + b)
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")      # read-only buffer: we never write through it
            t = torch.from_numpy(arr)
        if torch_dt == torch.bfloat16:
            t = t.view(torch.bfloat16)
        return t.reshape(shape)

    def close(self):
        try:
            self._mm.close()
        except BufferError:
            pass            # views are still alive; the map goes with them
        self._f.close()


def open_safetensors(path: str) -> SafetensorsFile:
    return SafetensorsFile(path)


def write_safetensors(path: str, tensors: dict, metadata: dict | None = None) -> None:
    """Write CPU tensors in name order; data offsets are 8-byte aligned by header padding."""
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    order = sorted(tensors.keys())
    for name in order:
        t = tensors[name]
        if t.dtype not in _TORCH_TO_NAME:
            raise SafetensorsError(f"cannot write tensor '{name}' of dtype {t.dtype}")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _TORCH_TO_NAME[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    raw = json.dumps(header, separators=(",", ":")).encode("utf-8")
    raw += b" " * ((8 - len(raw) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(raw)))
        f.write(raw)
        for name in order:
            t = tensors[name].detach().contiguous().cpu()
            if t.dtype == torch.bfloat16:
                t = t.view(torch.int16)
            f.write(t.numpy().tobytes())
