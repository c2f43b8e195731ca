"""Entry point of the tensor-core attention kernels (csrc/attn_mma.cu), which are compiled
once for each head size a model uses."""
from __future__ import annotations

from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from . import build
from .ops import KernelError, _check, _ptr, _stream, sm_count

SOURCE = "attn_mma.cu"
import os as _os
SLICE_FACTOR = int(_os.environ.get("ULTIMA_SLICE_FACTOR", "2"))
SLICE_CAP = int(_os.environ.get("ULTIMA_SLICE_CAP", "16"))
_libs: dict = {}


def target(head_dim: int):
    extra = tuple(x for x in _os.environ.get("ULTIMA_ATTN_DEFINES", "").split(",") if x)
    return (SOURCE, (f"HEAD_DIM={int(head_dim)}",) + extra)


def lib(head_dim: int):
    L = _libs.get(head_dim)
    if L is None:
        L = build.load(*target(head_dim))
        L.ub_attn_mma.argtypes = [c_int, c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p,
                                  c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                  c_float, c_int, c_void_p, c_void_p, c_void_p]
        L.ub_attn_mma.restype = c_int
        L.ub_attn_head_dim.restype = c_int
        if L.ub_attn_head_dim() != head_dim:
            raise KernelError(f"attention library was built for head size {L.ub_attn_head_dim()}, not {head_dim}")
        if head_dim % 64 == 0:
            L.ub_attn_map_kv.argtypes = [c_void_p, c_void_p, c_longlong, c_int]
            L.ub_attn_map_kv.restype = c_int
            L.ub_attn_decode_tma.argtypes = [c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_longlong, c_void_p,
                                             c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                             c_float, c_int, c_void_p, c_void_p, c_void_p, c_void_p]
            L.ub_attn_decode_tma.restype = c_int
            L.ub_attn_decode_tma_qkv.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_longlong, c_void_p, c_void_p,
                                                 c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_void_p, c_longlong,
                                                 c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                                 c_int, c_float, c_int, c_void_p, c_void_p, c_void_p, c_void_p]
            L.ub_attn_decode_tma_qkv.restype = c_int
        _libs[head_dim] = L
    return L


TC_SOURCE = "attn_tcgen05.cu"
_tc_libs: dict = {}
_tc_maps: dict = {}
USE_TCGEN05 = _os.environ.get("ULTIMA_ATTN_TCGEN05", "1") != "0"
USE_TCGEN05_DECODE = _os.environ.get("ULTIMA_ATTN_TCGEN05_DECODE", "0") != "0"
USE_TMA_DECODE = _os.environ.get("ULTIMA_ATTN_TMA_DECODE", "1") != "0"
# prompts on the tcgen05 kernel: 1 = 256 rows a CTA when that still gives every SM a CTA, 0 = always 128 rows
# a CTA, 2 = always 256
WIDE = int(_os.environ.get("ULTIMA_ATTN_WIDE", "1"))


def tc_target(head_dim: int):
    return (TC_SOURCE, (f"HEAD_DIM={int(head_dim)}",))


def tc_lib(head_dim: int):
    L = _tc_libs.get(head_dim)
    if L is None:
        L = build.load(*tc_target(head_dim))
        L.ub_attn_tc_map_q.argtypes = [c_void_p, c_void_p, c_longlong, c_int, c_longlong, c_int]
        L.ub_attn_tc_map_q.restype = c_int
        L.ub_attn_tc_map_kv.argtypes = [c_void_p, c_void_p, c_longlong, c_int]
        L.ub_attn_tc_map_kv.restype = c_int
        L.ub_attn_tc.argtypes = [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p,
                                 c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p,
                                 c_void_p, c_void_p, c_void_p]
        L.ub_attn_tc.restype = c_int
        L.ub_attn_tc_set_wide.argtypes = [c_int]
        L.ub_attn_tc_set_wide.restype = None
        L.ub_attn_tc_set_wide(WIDE)
        _tc_libs[head_dim] = L
    return L


def set_wide(mode: int) -> None:
    """Choose between the two prompt kernels (see ``WIDE``) in every library loaded so far and later."""
    global WIDE
    WIDE = int(mode)
    for L in _tc_libs.values():
        L.ub_attn_tc_set_wide(WIDE)


def tcgen05_fits(head_dim: int, n_heads: int, n_kv_heads: int) -> bool:
    """The tcgen05 kernel: head sizes 64 and 128, groups of up to 128 query heads a KV head."""
    return USE_TCGEN05 and head_dim in (64, 128) and n_heads // n_kv_heads <= 128


def _tc_map(key, make):
    import ctypes
    hit = _tc_maps.get(key)
    if hit is not None:
        return hit[1]
    raw = ctypes.create_string_buffer(128 + 64)
    addr = (ctypes.addressof(raw) + 63) & ~63
    rc = make(addr)
    if rc != 0:
        raise KernelError(f"tensor map for attention could not be made (code {rc})")
    if len(_tc_maps) > 1024:
        _tc_maps.clear()
    _tc_maps[key] = (raw, addr)
    return addr


def run_tcgen05(q, kv, out, batch, n_heads, n_kv_heads, head_dim, scale, rt, decode: bool, n_slices: int = 1):
    L = tc_lib(head_dim)
    group = n_heads // n_kv_heads
    T = q.shape[0]
    mq = _tc_map(("q", q.data_ptr(), T, n_heads, q.stride(0), group, head_dim),
                 lambda a: L.ub_attn_tc_map_q(a, q.data_ptr(), T, n_heads, q.stride(0), group))
    mk = _tc_map(("kv", kv.k.data_ptr(), kv.k.shape[0], n_kv_heads, head_dim),
                 lambda a: L.ub_attn_tc_map_kv(a, kv.k.data_ptr(), kv.k.shape[0], n_kv_heads))
    mv = _tc_map(("kv", kv.v.data_ptr(), kv.v.shape[0], n_kv_heads, head_dim),
                 lambda a: L.ub_attn_tc_map_kv(a, kv.v.data_ptr(), kv.v.shape[0], n_kv_heads))
    part_o = part_ml = None
    if decode and n_slices > 1:
        part_o = rt.arena.alloc((batch.n_seqs, n_heads, n_slices, head_dim), torch.float32)
        part_ml = rt.arena.alloc((batch.n_seqs, n_heads, n_slices, 2), torch.float32)
    rc = L.ub_attn_tc(1 if decode else 0, mq, mk, mv, _ptr(out), out.stride(0), _ptr(batch.seq_start),
                      _ptr(batch.seq_before), _ptr(kv.table), kv.table.shape[1], kv.ring, kv.page, batch.n_seqs,
                      batch.max_new, n_heads, n_kv_heads, int(kv.window or 0), float(scale), n_slices,
                      _ptr(part_o), _ptr(part_ml), _ptr(rt.status[1:2]), _stream())
    _check(rc, "attn_tc")


def accepts(q, kv, head_dim, n_heads, n_kv_heads) -> bool:
    return (q.dtype == torch.bfloat16 and kv.k.dtype == torch.bfloat16 and head_dim % 16 == 0
            and 16 <= head_dim <= 256 and kv.page == 64 and q.stride(1) == 1 and q.stride(0) % 8 == 0
            and q.data_ptr() % 16 == 0)


def decode_slices(n_seqs: int, n_kv_heads: int, longest: int, window, per_sm: int = SLICE_FACTOR,
                  n_sms: int | None = None) -> int:
    """Slices of the key range, so that a decode step with few sequences still fills the GPU
    (``per_sm`` CTAs an SM; ``n_sms``: the device's multiprocessors, asked of it when not given)."""
    span = longest if not window else min(longest, window + 64)
    tiles = max(1, -(-span // 64))
    ctas = n_seqs * n_kv_heads
    want = -(-per_sm * (n_sms or sm_count()) // ctas)
    n = max(1, min(want, tiles, SLICE_CAP))
    return 1 << (n.bit_length() - 1)            # a power of two: few distinct captured graphs


FUSE_QKV = _os.environ.get("ULTIMA_ATTN_FUSE_QKV", "1") != "0"


def decode_from_qkv(qkv, q_norm, k_norm, cos, sin, eps, kv, out, batch, n_heads, n_kv_heads, head_dim, scale, rt,
                    slices: int | None = None, force: bool = False) -> bool:
    """A step of one token a sequence, straight from the fused projection's float32 partial results
    ``qkv`` [parts, T, (heads + 2 kv heads) * head size]: the attention kernel sums them, norms and
    rotates its own query heads and the new key, and writes the new key and value into the cache
    (when this layer owns it).  False: the case is not this kernel's (the caller prepares q and
    calls ``attention``)."""
    if not (FUSE_QKV or force) or not (USE_TMA_DECODE or force):
        return False
    group = n_heads // n_kv_heads
    if not (batch.max_new == 1 and group <= 16 and head_dim in (64, 128, 256) and qkv.dim() == 3
            and qkv.dtype == torch.float32 and qkv.is_contiguous() and kv.k.dtype == torch.bfloat16
            and kv.k.is_contiguous() and kv.v.is_contiguous() and kv.page == 64
            and out.dtype == torch.bfloat16 and out.stride(1) == 1 and qkv.stride(0) % 4 == 0
            and qkv.shape[2] == (n_heads + 2 * n_kv_heads) * head_dim):
        return False
    if USE_TCGEN05_DECODE and not force:
        return False
    for t in (q_norm, k_norm, cos, sin):
        if t is not None and not (t.dtype == torch.float32 and t.is_contiguous() and t.data_ptr() % 16 == 0):
            return False
    L = lib(head_dim)
    n_slices = slices or decode_slices(batch.n_seqs, n_kv_heads, batch.max_after, kv.window)
    part_o = part_ml = None
    if n_slices > 1:
        part_o = rt.arena.alloc((batch.n_seqs, n_heads, n_slices, head_dim), torch.float32)
        part_ml = rt.arena.alloc((batch.n_seqs, n_heads, n_slices, 2), torch.float32)
    mk = _tc_map(("kvd", kv.k.data_ptr(), kv.k.shape[0], n_kv_heads, head_dim),
                 lambda a: L.ub_attn_map_kv(a, kv.k.data_ptr(), kv.k.shape[0], n_kv_heads))
    mv = _tc_map(("kvd", kv.v.data_ptr(), kv.v.shape[0], n_kv_heads, head_dim),
                 lambda a: L.ub_attn_map_kv(a, kv.v.data_ptr(), kv.v.shape[0], n_kv_heads))
    own = bool(kv.owner)
    rc = L.ub_attn_decode_tma_qkv(mk, mv, _ptr(qkv), qkv.shape[0], qkv.stride(0), _ptr(q_norm), _ptr(k_norm),
                                  _ptr(cos), _ptr(sin), float(eps), _ptr(kv.k) if own else None,
                                  _ptr(kv.v) if own else None, _ptr(out), out.stride(0), _ptr(batch.seq_start),
                                  _ptr(batch.seq_before), _ptr(kv.table), kv.table.shape[1], kv.ring, kv.page,
                                  batch.n_seqs, n_heads, n_kv_heads, int(kv.window or 0), float(scale), n_slices,
                                  _ptr(part_o), _ptr(part_ml), _ptr(rt.status[1:2]), _stream())
    _check(rc, "attn_decode_tma_qkv")
    return True


def attention(q, kv, out, batch, n_heads, n_kv_heads, head_dim, scale, rt, slices: int | None = None,
              kernel: str | None = None):
    """kernel: None picks (tcgen05 for prompts where it fits, mma.sync otherwise); "mma" forces the latter."""
    L = lib(head_dim)
    assert out.dtype == torch.bfloat16 and out.stride(1) == 1
    group = n_heads // n_kv_heads
    decode = batch.max_new == 1 and group <= 16
    tc_ok = (kernel != "mma" and tcgen05_fits(head_dim, n_heads, n_kv_heads) and out.stride(0) % 8 == 0
             and out.data_ptr() % 16 == 0 and kv.k.is_contiguous() and kv.v.is_contiguous())
    if tc_ok and not decode:
        return run_tcgen05(q, kv, out, batch, n_heads, n_kv_heads, head_dim, scale, rt, False)
    if tc_ok and decode and (USE_TCGEN05_DECODE or kernel == "tc"):
        n = slices or decode_slices(batch.n_seqs, n_kv_heads, batch.max_after, kv.window, per_sm=1)
        return run_tcgen05(q, kv, out, batch, n_heads, n_kv_heads, head_dim, scale, rt, True, n)
    part_o = part_ml = None
    n_slices = 1
    tma = (decode and head_dim % 64 == 0 and kernel in (None, "tma") and (USE_TMA_DECODE or kernel == "tma")
           and kv.k.is_contiguous() and kv.v.is_contiguous())
    if decode:
        n_slices = slices or decode_slices(batch.n_seqs, n_kv_heads, batch.max_after, kv.window)
        if n_slices > 1:
            part_o = rt.arena.alloc((batch.n_seqs, n_heads, n_slices, head_dim), torch.float32)
            part_ml = rt.arena.alloc((batch.n_seqs, n_heads, n_slices, 2), torch.float32)
    if tma:
        mk = _tc_map(("kvd", kv.k.data_ptr(), kv.k.shape[0], n_kv_heads, head_dim),
                     lambda a: L.ub_attn_map_kv(a, kv.k.data_ptr(), kv.k.shape[0], n_kv_heads))
        mv = _tc_map(("kvd", kv.v.data_ptr(), kv.v.shape[0], n_kv_heads, head_dim),
                     lambda a: L.ub_attn_map_kv(a, kv.v.data_ptr(), kv.v.shape[0], n_kv_heads))
        rc = L.ub_attn_decode_tma(mk, mv, _ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(batch.seq_start),
                                  _ptr(batch.seq_before), _ptr(kv.table), kv.table.shape[1], kv.ring, kv.page,
                                  batch.n_seqs, n_heads, n_kv_heads, int(kv.window or 0), float(scale), n_slices,
                                  _ptr(part_o), _ptr(part_ml), _ptr(rt.status[1:2]), _stream())
        return _check(rc, "attn_decode_tma")
    rc = L.ub_attn_mma(1 if decode else 0, _ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(kv.k), _ptr(kv.v),
                       _ptr(batch.seq_start), _ptr(batch.seq_before), _ptr(kv.table), kv.table.shape[1], kv.ring,
                       kv.page, batch.n_seqs, batch.max_new, n_heads, n_kv_heads, int(kv.window or 0), float(scale),
                       n_slices, _ptr(part_o), _ptr(part_ml), _stream())
    _check(rc, "attn_mma")
