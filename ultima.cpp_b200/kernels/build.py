"""Compiling the CUDA sources of ``csrc/`` for sm_100a and loading them.

Each source becomes one shared library with a C interface, built with nvcc at its first
use and kept beside the sources (``csrc/_build``; a per-user folder under the system's
temporary directory if that is not writable).  The file name carries a hash of the source,
the shared header and the flags, so a stale library is never loaded.  Nothing here needs a
home directory or a network.  While nvcc runs, a line is printed every few seconds.

There is no fallback: if a library cannot be built or loaded, the caller gets an error.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time

_HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(os.path.dirname(_HERE), "csrc")
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
BASE_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-shared", "-Xcompiler", "-fPIC",
              "-Xcompiler", "-fvisibility=hidden"]


class BuildError(RuntimeError):
    pass


_lock = threading.Lock()
_loaded: dict[str, ctypes.CDLL] = {}


def _say(msg: str) -> None:
    print(f"[ultima_b200] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for cand in (os.environ.get("ULTIMA_NVCC"), shutil.which("nvcc"),
                 os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"),
                 "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("nvcc not found (looked at $ULTIMA_NVCC, PATH, $CUDA_HOME/bin, "
                     "/usr/local/cuda/bin); the CUDA kernels cannot be built")


def build_dir() -> str:
    d = os.path.join(CSRC, "_build")
    try:
        os.makedirs(d, exist_ok=True)
        probe = os.path.join(d, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return d
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"ultima_b200_build_{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def _headers() -> list[str]:
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h")))


def _target(source: str, defines: tuple) -> tuple[str, list[str]]:
    src = os.path.join(CSRC, source)
    if not os.path.isfile(src):
        raise BuildError(f"kernel source '{src}' is missing")
    flags = BASE_FLAGS + ARCH_FLAGS + [f"-D{d}" for d in defines]
    h = hashlib.sha1()
    for p in [src] + _headers():
        with open(p, "rb") as f:
            h.update(f.read())
    h.update(" ".join(flags).encode())
    tag = "".join(c if c.isalnum() else "_" for c in "_".join(defines))
    stem = os.path.splitext(source)[0] + (("_" + tag) if tag else "")
    return f"{stem}-{h.hexdigest()[:12]}.so", flags


def ensure_built(targets: list[tuple]) -> dict:
    """targets: [(source, (defines...)), ...] -> {(source, defines): path}; missing ones are
    compiled side by side."""
    out, jobs = {}, []
    bdir = build_dir()
    for source, defines in targets:
        defines = tuple(defines)
        name, flags = _target(source, defines)
        path = os.path.join(bdir, name)
        out[(source, defines)] = path
        if not os.path.isfile(path):
            jobs.append((source, defines, path, flags))
    if not jobs:
        return out
    nvcc = find_nvcc()
    procs = []
    t0 = time.time()
    for source, defines, path, flags in jobs:
        tmp = f"{path}.{os.getpid()}.tmp"
        cmd = [nvcc] + flags + ["-o", tmp, os.path.join(CSRC, source)]
        _say(f"compiling {source} {' '.join(defines)} for sm_100a ...")
        procs.append((source, path, tmp, subprocess.Popen(
            cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, cwd=bdir)))
    last = time.time()
    pending = list(procs)
    errors = []
    while pending:
        for item in list(pending):
            source, path, tmp, p = item
            if p.poll() is None:
                continue
            pending.remove(item)
            log = p.stdout.read()
            if p.returncode != 0:
                errors.append(f"nvcc failed on {source}:\n{log}")
                continue
            os.replace(tmp, path)
            _drop_stale(path)
            _say(f"built {os.path.basename(path)} after {time.time() - t0:.0f} s")
        if pending and time.time() - last > 5:
            last = time.time()
            _say(f"still compiling {', '.join(i[0] for i in pending)} ({time.time() - t0:.0f} s)")
        if pending:
            time.sleep(0.2)
    if errors:
        raise BuildError("\n".join(errors))
    return out


def _drop_stale(path: str) -> None:
    """Remove earlier builds of the same source and defines (other hashes)."""
    d, name = os.path.split(path)
    stem = name.rsplit("-", 1)[0]
    for f in os.listdir(d):
        if f != name and f.endswith(".so") and f.rsplit("-", 1)[0] == stem:
            try:
                os.remove(os.path.join(d, f))
            except OSError:
                pass


def load(source: str, defines: tuple = ()) -> ctypes.CDLL:
    key = source + "|" + ",".join(defines)
    with _lock:
        if key in _loaded:
            return _loaded[key]
        path = ensure_built([(source, tuple(defines))])[(source, tuple(defines))]
        try:
            lib = ctypes.CDLL(path)
        except OSError as e:
            raise BuildError(f"cannot load {path}: {e}") from e
        _loaded[key] = lib
        return lib


def prebuild(targets: list[tuple]) -> None:
    """Compile several libraries at once (their nvcc runs overlap), then load them."""
    with _lock:
        ensure_built([(s, tuple(d)) for s, d in targets])
    for s, d in targets:
        load(s, tuple(d))
