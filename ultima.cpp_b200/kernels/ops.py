"""Python entry points of the CUDA kernels.  Each takes torch tensors on the GPU, checks
what the kernel assumes, and launches on torch's current stream.  There is no other
implementation behind them: on a machine without the GPU or the compiler they raise.
"""
from __future__ import annotations

from ctypes import c_float, c_int, c_longlong, c_ulonglong, c_void_p

import numpy as np
import torch

from . import build

F32, BF16 = 0, 1
EPI_STORE, EPI_ADD, EPI_SWIGLU, EPI_SWIGLU_IL = 0, 1, 2, 3
MAX_HEAD_DIM = 256          # the largest head size the attention and q/k preparation kernels take


class KernelError(RuntimeError):
    pass


_sm_counts: dict = {}


def sm_count(device=None) -> int:
    """Streaming multiprocessors of the device (the current one by default), asked of the device once.
    Slice counts, K splits and the choice between kernels follow it."""
    if device is None:
        n = _sm_counts.get(None)
        if n is not None:
            return n
    if not torch.cuda.is_available():
        raise KernelError("no CUDA device: the number of multiprocessors cannot be asked")
    idx = torch.cuda.current_device() if device is None else torch.device(device).index or 0
    n = _sm_counts.get(idx)
    if n is None:
        n = _sm_counts[idx] = int(torch.cuda.get_device_properties(idx).multi_processor_count)
    if device is None:
        _sm_counts[None] = n            # (one process drives one GPU: the current device does not change)
    return n


def _code(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16 tensors, got {t.dtype}")


def _ptr(t):
    return 0 if t is None else t.data_ptr()


# The current stream's handle is asked for at every launch: through the raw accessor that torch's own
# extensions use (a few hundred nanoseconds) where it exists, not through the Stream object (microseconds).
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream() -> int:
    if _raw_stream is None or _raw_device is None:
        return torch.cuda.current_stream().cuda_stream
    return _raw_stream(_raw_device())


def _check(rc: int, what: str) -> None:
    if rc == 0:
        return
    if rc == -1:
        raise KernelError(f"{what}: an argument is outside what the kernel takes")
    if rc == -2:
        raise KernelError(f"{what}: this combination of element types is not built")
    raise KernelError(f"{what}: CUDA error {rc} at launch")


def _need_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise KernelError("kernels run on CUDA tensors only; there is no CPU path")


_sigs_done = set()


def _lib(source: str, defines=()):
    lib = build.load(source, tuple(defines))
    key = (source, tuple(defines))
    if key not in _sigs_done:
        _declare(lib, source)
        _sigs_done.add(key)
    return lib


def _declare(lib, source: str) -> None:
    P, I, L, F, U = c_void_p, c_int, c_longlong, c_float, c_ulonglong
    sigs = {
        "basic.cu": {
            "ub_embed": [P, I, P, P, I, I, I, P, P],
            "ub_rmsnorm": [P, P, P, P, I, I, I, F, P],
            "ub_qk_prepare": [P, I, I, L, P, I, L, P, P, P, P, P, P, P, P, I, P, I, I, I, I, I, I, I, F, I, I, I, P, P, L, P],
            "ub_rotate_pairs": [P, I, L, I, I, I, P, P, P, I, I, P],
            "ub_kv_write": [P, P, I, L, P, P, P, P, I, P, I, I, I, I, I, I, P],
            "ub_silu_mul": [P, I, I, L, P, I, I, I, P],
            "ub_convert": [P, I, P, I, L, P],
            "ub_add_into": [P, P, I, L, P],
            "ub_fill_normal": [P, I, L, U, F, F, P],
        },
        "gemm_simt.cu": {"ub_gemm_simt": [P, I, P, P, I, P, I, I, I, I, L, L, L, I, P]},
        "attn_simple.cu": {"ub_attn_simple": [P, L, I, P, P, I, P, L, P, P, P, I, I, I, I, I, I, I, I, F, P]},
        "sampling.cu": {"ub_sample": [P, L, P, I, I, P, P, P, P, P, U, P, P, I, P], "ub_sample_params_size": []},
    }.get(source, {})
    for name, args in sigs.items():
        fn = getattr(lib, name)
        fn.argtypes = args
        fn.restype = c_int


# ---------------------------------------------------------------------------------------
def embed(table, ids, out, status):
    """out[t, :] = table[ids[t], :] as float32; a bad id raises ``status`` (int32[1])."""
    _need_cuda(table, ids, out, status)
    T, width = out.shape
    assert out.dtype == torch.float32 and ids.dtype == torch.int32 and out.is_contiguous()
    assert table.is_contiguous() and table.shape[1] == width
    _check(_lib("basic.cu").ub_embed(_ptr(table), _code(table), _ptr(ids), _ptr(out), T, width,
                                     table.shape[0], _ptr(status), _stream()), "embed")


def rmsnorm(x, weight, out, eps, rows=None):
    """out[r, :] = x[rows[r] or r, :] * weight / sqrt(mean(x^2) + eps); x float32."""
    _need_cuda(x, weight, out, rows)
    assert x.dtype == torch.float32 and weight.dtype == torch.float32
    assert x.is_contiguous() and out.is_contiguous() and weight.is_contiguous()
    n, width = out.shape
    assert x.shape[1] == width and weight.numel() == width
    if rows is not None:
        assert rows.dtype == torch.int32 and rows.numel() == n
    _check(_lib("basic.cu").ub_rmsnorm(_ptr(x), _ptr(rows), _ptr(weight), _ptr(out), _code(out), n,
                                       width, float(eps), _stream()), "rmsnorm")


def qk_prepare(qkv, q_weight, k_weight, cos, sin, tok_pos, tok_seq, k_cache, v_cache, table,
               ring, page, n_heads, n_kv_heads, head_dim, eps, write_kv=True, q_out=None,
               rotary_dim=None, interleaved=False, kv_out=None):
    """Per-head norm and rotation of q and k, and the write of k, v into the cache.

    qkv: [T, (heads + 2 kv heads) * head size], or [parts, T, ...] whose sum over parts it is
    (slices of K of the projection).  q goes to ``q_out`` ([T, heads * head size], any row stride),
    or back into qkv's q columns when q_out is None (one part only).  cos, sin: [positions,
    rotary_dim / 2]; the first ``rotary_dim`` columns of a head (default: all) are rotated, in pairs
    (j, j + rotary_dim / 2) or, ``interleaved``, (2j, 2j + 1).  ``kv_out`` = (k, v), each
    [T, kv heads * head size] with q_out's element type and one row stride: keys and values go
    there instead of into the cache (see ``kv_write``)."""
    _need_cuda(qkv, k_cache, v_cache, table)
    width = (n_heads + 2 * n_kv_heads) * head_dim
    if qkv.dim() == 3:
        n_parts, T = qkv.shape[0], qkv.shape[1]
        part_stride = qkv.stride(0)
        assert qkv.shape[2] == width and qkv.stride(1) == width and qkv.stride(2) == 1
        assert q_out is not None
    else:
        n_parts, T, part_stride = 1, qkv.shape[0], 0
        assert qkv.is_contiguous() and qkv.shape[1] == width
    if q_out is None:
        q_out = qkv
    assert q_out.stride(1) == 1 and q_out.shape[0] == T
    assert table.dtype == torch.int32 and table.dim() == 2 and table.is_contiguous()
    for v in (q_weight, k_weight, cos, sin):
        assert v is None or (v.dtype == torch.float32 and v.is_contiguous())
    rd = int(rotary_dim) if rotary_dim is not None else head_dim
    if cos is not None:
        if rd % 2 or not (2 <= rd <= head_dim):
            raise KernelError(f"qk_prepare: rotary size {rd} must be even and at most the head size {head_dim}")
        assert cos.shape[1] == rd // 2 and sin.shape == cos.shape
    k_out = v_out = None
    kv_stride = 0
    if kv_out is not None:
        k_out, v_out = kv_out
        assert k_out.dtype == q_out.dtype == v_out.dtype and k_out.stride(1) == 1 and v_out.stride(1) == 1
        assert k_out.stride(0) == v_out.stride(0) and k_out.shape == v_out.shape == (T, n_kv_heads * head_dim)
        kv_stride = k_out.stride(0)
    _check(_lib("basic.cu").ub_qk_prepare(
        _ptr(qkv), _code(qkv), n_parts, part_stride, _ptr(q_out), _code(q_out), q_out.stride(0),
        _ptr(q_weight), _ptr(k_weight), _ptr(cos), _ptr(sin), _ptr(tok_pos),
        _ptr(tok_seq), _ptr(k_cache), _ptr(v_cache), _code(k_cache), _ptr(table), table.shape[1],
        ring, page, T, n_heads, n_kv_heads, head_dim, float(eps), 1 if write_kv else 0,
        rd, 1 if interleaved else 0, _ptr(k_out), _ptr(v_out), kv_stride, _stream()),
        "qk_prepare")


def rotate_pairs(x, cos, sin, tok_pos, rotary_dim=None, interleaved=False):
    """Rotate, in place, pairs of the first ``rotary_dim`` columns of every head of x [T, heads,
    head size] (heads side by side in a row, any row stride) by the angles of each token's position."""
    _need_cuda(x, cos, sin, tok_pos)
    T, n_heads, hd = x.shape
    assert x.stride(2) == 1 and x.stride(1) == hd and cos.dtype == torch.float32 and cos.is_contiguous()
    rd = int(rotary_dim) if rotary_dim is not None else hd
    assert cos.shape[1] == rd // 2 and sin.shape == cos.shape and tok_pos.dtype == torch.int32
    _check(_lib("basic.cu").ub_rotate_pairs(_ptr(x), _code(x), x.stride(0), T, n_heads, hd, _ptr(cos), _ptr(sin),
                                            _ptr(tok_pos), rd, 1 if interleaved else 0, _stream()), "rotate_pairs")


def kv_write(k, v, tok_pos, tok_seq, k_cache, v_cache, table, ring, page, n_kv_heads, head_dim):
    """k, v [T, kv heads * head size] (one row stride) into the paged cache at each token's position."""
    _need_cuda(k, v, k_cache, v_cache, table)
    T = k.shape[0]
    assert k.shape == v.shape == (T, n_kv_heads * head_dim) and k.stride(1) == 1 and v.stride(1) == 1
    assert k.stride(0) == v.stride(0) and k.dtype == v.dtype
    assert table.dtype == torch.int32 and table.dim() == 2 and table.is_contiguous()
    _check(_lib("basic.cu").ub_kv_write(_ptr(k), _ptr(v), _code(k), k.stride(0), _ptr(tok_pos), _ptr(tok_seq), _ptr(k_cache),
                                        _ptr(v_cache), _code(k_cache), _ptr(table), table.shape[1], ring, page, T,
                                        n_kv_heads, head_dim, _stream()), "kv_write")


def silu_mul(gate_up, out):
    """out[t, f] = silu(g[t, f]) * g[t, F + f], g being gate_up ([T, 2F]) or the sum over the first
    axis of gate_up ([parts, T, 2F])."""
    _need_cuda(gate_up, out)
    T, F = out.shape
    if gate_up.dim() == 3:
        n_parts, part_stride = gate_up.shape[0], gate_up.stride(0)
        assert gate_up.shape[1:] == (T, 2 * F) and gate_up.stride(1) == 2 * F and gate_up.stride(2) == 1
    else:
        n_parts, part_stride = 1, 0
        assert gate_up.shape == (T, 2 * F) and gate_up.is_contiguous()
    assert out.is_contiguous()
    _check(_lib("basic.cu").ub_silu_mul(_ptr(gate_up), _code(gate_up), n_parts, part_stride, _ptr(out),
                                        _code(out), T, F, _stream()), "silu_mul")


def convert(src, dst):
    _need_cuda(src, dst)
    assert src.numel() == dst.numel() and src.is_contiguous() and dst.is_contiguous()
    _check(_lib("basic.cu").ub_convert(_ptr(src), _code(src), _ptr(dst), _code(dst), src.numel(),
                                       _stream()), "convert")


def add_into(acc, src):
    _need_cuda(acc, src)
    assert acc.dtype == torch.float32 and acc.numel() == src.numel()
    assert acc.is_contiguous() and src.is_contiguous()
    _check(_lib("basic.cu").ub_add_into(_ptr(acc), _ptr(src), _code(src), acc.numel(), _stream()),
           "add_into")


def fill_normal(out, seed: int, shift: float, std: float):
    _need_cuda(out)
    assert out.is_contiguous()
    _check(_lib("basic.cu").ub_fill_normal(_ptr(out), _code(out), out.numel(), seed & (2**64 - 1),
                                           float(shift), float(std), _stream()), "fill_normal")


def gemm_simt(a, w, out, epilogue=EPI_STORE, w2=None):
    """out[t, n] (=, +=) sum_k a[t, k] w[n, k] on the CUDA cores with float32 FMA;
    EPI_SWIGLU: out = silu(a w^T) * (a w2^T)."""
    _need_cuda(a, w, out, w2)
    M, K = a.shape
    N = w.shape[0]
    assert w.shape[1] == K and out.shape == (M, N)
    assert a.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
    if w2 is not None:
        assert w2.shape == w.shape and w2.dtype == w.dtype and w2.stride() == w.stride()
    _check(_lib("gemm_simt.cu").ub_gemm_simt(
        _ptr(a), _code(a), _ptr(w), _ptr(w2), _code(w), _ptr(out), _code(out), M, N, K,
        a.stride(0), w.stride(0), out.stride(0), epilogue, _stream()), "gemm_simt")


def attn_simple(q, k_cache, v_cache, out, tok_pos, tok_seq, table, ring, page, n_heads,
                n_kv_heads, head_dim, window, scale):
    """Attention of every token of the step over its sequence's cached keys and values."""
    _need_cuda(q, k_cache, v_cache, out, table)
    T = q.shape[0]
    assert q.stride(1) == 1 and out.stride(1) == 1 and q.dtype == out.dtype
    assert table.dtype == torch.int32 and table.dim() == 2 and table.is_contiguous()
    _check(_lib("attn_simple.cu").ub_attn_simple(
        _ptr(q), q.stride(0), _code(q), _ptr(k_cache), _ptr(v_cache), _code(k_cache), _ptr(out),
        out.stride(0), _ptr(tok_pos), _ptr(tok_seq), _ptr(table), table.shape[1], ring, page, T,
        n_heads, n_kv_heads, head_dim, int(window or 0), float(scale), _stream()), "attn_simple")


# ---------------------------------------------------------------------------------------
SAMPLE_DTYPE = np.dtype([
    ("temperature", "<f4"), ("top_p", "<f4"), ("min_p", "<f4"), ("rep_penalty", "<f4"),
    ("freq_penalty", "<f4"), ("presence_penalty", "<f4"), ("dry_multiplier", "<f4"),
    ("dry_base", "<f4"), ("top_k", "<i4"), ("repeat_last_n", "<i4"), ("dry_last_n", "<i4"),
    ("dry_allowed_len", "<i4"), ("n_recent", "<i4"), ("recent_offset", "<i4"), ("n_bias", "<i4"),
    ("bias_offset", "<i4"), ("seed", "<u8"), ("counter", "<u8")])


def sample(logits, work, params_dev, recent, bias_ids, bias_vals, out_ids, counter_add: int = 0,
           hist=None, hist_len=None):
    """One token id for each row of float32 ``logits``; ``params_dev`` holds one record of
    SAMPLE_DTYPE a row (as bytes on the device); ``counter_add`` is added to every row's counter.
    ``hist`` [rings, capacity] int32 and ``hist_len`` [rings] int32: rings of recent tokens that stay on
    the device; a row whose record has n_recent < 0 reads ring ``recent_offset`` and appends its token."""
    _need_cuda(logits, work, params_dev, out_ids)
    lib = _lib("sampling.cu")
    assert lib.ub_sample_params_size() == SAMPLE_DTYPE.itemsize
    n, V = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(1) == 1
    assert work is None or (work.dtype == torch.float32 and work.is_contiguous() and work.numel() >= n * V)
    assert out_ids.dtype == torch.int32 and out_ids.numel() >= n
    cap = 0
    if hist is not None:
        assert hist.dtype == torch.int32 and hist.dim() == 2 and hist.is_contiguous()
        assert hist_len is not None and hist_len.dtype == torch.int32 and hist_len.numel() >= hist.shape[0]
        cap = hist.shape[1]
    _check(lib.ub_sample(_ptr(logits), logits.stride(0), _ptr(work), n, V, _ptr(params_dev),
                         _ptr(recent), _ptr(bias_ids), _ptr(bias_vals), _ptr(out_ids), int(counter_add),
                         _ptr(hist), _ptr(hist_len), cap, _stream()),
           "sample")
