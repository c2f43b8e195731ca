"""Entry point of the tcgen05 matrix product (csrc/gemm_tcgen05.cu): which calls it takes,
which token tile and K split it uses, and the tensor maps it needs (made once for each matrix
and kept)."""
from __future__ import annotations

import ctypes
import os
from ctypes import c_int, c_longlong, c_void_p

import torch

from . import build
from .ops import EPI_ADD, EPI_STORE, EPI_SWIGLU, EPI_SWIGLU_IL, BF16, F32, KernelError, _check, _ptr, _stream, sm_count

SOURCE = "gemm_tcgen05.cu"
_lib = None
_maps: dict = {}


def lib():
    global _lib
    if _lib is None:
        L = build.load(SOURCE)
        L.ub_tmap_bf16_2d.argtypes = [c_void_p, c_void_p, c_longlong, c_longlong, c_longlong, c_int]
        L.ub_tmap_bf16_2d.restype = c_int
        L.ub_gemm_tc.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_longlong, c_longlong,
                                 c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p]
        L.ub_gemm_tc.restype = c_int
        L.ub_gemm_tc_pair.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_longlong, c_int, c_int, c_int, c_int,
                                      c_void_p, c_void_p]
        L.ub_gemm_tc_pair.restype = c_int
        L.ub_gemm_tc_set_pdl.argtypes = [c_int]
        L.ub_gemm_tc_set_pdl.restype = None
        import os
        if os.environ.get("ULTIMA_PDL", "1") == "0":       # for measurements: ordinary launches
            L.ub_gemm_tc_set_pdl(0)
        L.ub_gemm_tc_set_persistent.argtypes = [c_int]
        L.ub_gemm_tc_set_persistent.restype = None
        if os.environ.get("ULTIMA_PERSISTENT", "1") == "0":   # for measurements: one tile a CTA
            L.ub_gemm_tc_set_persistent(0)
        L.ub_gemm_tc_set_share_tail.argtypes = [c_int]
        L.ub_gemm_tc_set_share_tail.restype = None
        if os.environ.get("ULTIMA_SHARE_TAIL", "1") == "0":   # for measurements: whole tiles only
            L.ub_gemm_tc_set_share_tail(0)
        _lib = L
    return _lib


def _tmap_entry(t: torch.Tensor, box_rows: int):
    """(the buffer that holds it, address) of a 64-byte aligned CUtensorMap on the host for the 2-D bfloat16
    matrix ``t``."""
    key = (t.data_ptr(), t.shape[0], t.shape[1], t.stride(0), box_rows)
    hit = _maps.get(key)
    if hit is not None:
        return hit
    raw = ctypes.create_string_buffer(128 + 64)
    addr = (ctypes.addressof(raw) + 63) & ~63
    rc = lib().ub_tmap_bf16_2d(addr, t.data_ptr(), t.shape[0], t.shape[1], t.stride(0), box_rows)
    if rc != 0:
        raise KernelError(f"tensor map for a [{t.shape[0]}, {t.shape[1]}] matrix with row stride "
                          f"{t.stride(0)} could not be made (code {rc})")
    if len(_maps) > 4096:
        _maps.clear()
    _maps[key] = (raw, addr)
    return _maps[key]


def _tmap(t: torch.Tensor, box_rows: int) -> int:
    return _tmap_entry(t, box_rows)[1]


def _ok_operand(t: torch.Tensor) -> bool:
    return (t.dtype == torch.bfloat16 and t.dim() == 2 and t.stride(1) == 1 and t.stride(0) % 8 == 0
            and t.data_ptr() % 16 == 0)


def accepts(a, w, out, epilogue, w2) -> bool:
    """bfloat16 operands whose rows start on 16-byte boundaries (K and row strides multiples of 8);
    anything else goes to the CUDA-core kernel."""
    if not (_ok_operand(a) and _ok_operand(w)) or a.shape[1] % 8 != 0:
        return False
    if epilogue == EPI_SWIGLU:
        return w2 is not None and _ok_operand(w2) and out.dtype == torch.bfloat16
    if epilogue == EPI_SWIGLU_IL:
        return out.dtype == torch.bfloat16 and w.shape[0] % 128 == 0
    if epilogue == EPI_ADD:
        return out.dtype == torch.float32
    return out.dtype in (torch.bfloat16, torch.float32)


def token_tile(T: int, epilogue: int) -> int:
    for bn in (16, 32, 64, 128):
        if T <= bn:
            return bn
    if epilogue == EPI_SWIGLU:
        return 128
    return 256 if T > 192 else 128


def cta_slots(bn: int, epilogue: int, n_sms: int | None = None) -> int:
    """CTAs of this kernel that the GPU holds at once: two an SM for token tiles of up to 64 (their
    shared-memory ring is kept to half an SM's), one otherwise.  ``n_sms``: the device's
    multiprocessors (asked of the current device when not given)."""
    n_sms = n_sms or sm_count()
    return 2 * n_sms if (bn <= 64 and epilogue != EPI_SWIGLU) else n_sms


def k_splits(T: int, N: int, K: int, bn: int, epilogue: int, n_sms: int | None = None) -> int:
    """Slices of K, so that a product with few tiles still fills the GPU, and never more CTAs than
    the GPU holds at once (a second wave would start only when the first has ended).  Only the
    add-into epilogue is split here (its slices meet in the float32 residual stream)."""
    if epilogue != EPI_ADD:
        return 1
    tiles = -(-N // 128) * -(-T // bn)
    nkb = -(-K // 64)
    slots = cta_slots(bn, epilogue, n_sms)
    if tiles * 2 > slots or nkb < 8:
        return 1
    s = max(1, min(slots // tiles, nkb // 4))
    per = -(-nkb // s)
    return -(-nkb // per)


USE_PAIRS = os.environ.get("ULTIMA_GEMM_PAIRS", "1") != "0"
PAIRS_MIN_TOKENS = 1024


def pairs(T: int, N: int, splits: int, epilogue: int, n_sms: int | None = None) -> bool:
    """Whether the product runs on pairs of CTAs (tiles of 256 weight rows by 256 tokens): many
    tokens, K whole, and at least one tile for every pair of SMs.  Up to 1,024 tokens the one-CTA kernels,
    which start before the kernel in front of them has ended, are the faster choice (measured on whole
    prompts: 11.07 against 11.45 ms at 768 tokens, 14.33 against 14.43 at 1,024; 22.3 against 21.4 at 1,536)."""
    if not USE_PAIRS or splits != 1 or epilogue == EPI_SWIGLU or T <= PAIRS_MIN_TOKENS:
        return False
    return -(-N // 256) * -(-T // 256) >= (n_sms or sm_count()) // 2


def gemm(a, w, out, epilogue, w2, rt, splits: int | None = None, bn: int | None = None, key=None):
    """out: [T, N]; for EPI_SWIGLU_IL [T, N / 2]; for EPI_STORE with ``splits`` > 1 a float32
    [splits, T, N] whose sum over the first axis is the product."""
    T, K = a.shape
    N = w.shape[0]
    assert w.shape[1] == K and out.stride(-1) == 1
    tile_given = bn is not None
    bn = bn or token_tile(T, epilogue)
    s = splits or k_splits(T, N, K, bn, epilogue)
    split_stride = 0
    if out.dim() == 3:
        assert epilogue == EPI_STORE and out.dtype == torch.float32 and out.shape == (s, T, N)
        split_stride, ldo = out.stride(0), out.stride(1)
    else:
        assert out.shape == (T, N // 2 if epilogue == EPI_SWIGLU_IL else N)
        assert s == 1 or epilogue == EPI_ADD
        ldo = out.stride(0)
    L = lib()
    if not tile_given and out.dim() == 2 and pairs(T, N, s, epilogue):
        fn, what = L.ub_gemm_tc_pair, "gemm_tc_pair"
        maps = (_tmap_entry(w, 128), _tmap_entry(a, 128))
        args = (maps[0][1], maps[1][1], _ptr(out), BF16 if out.dtype == torch.bfloat16 else F32,
                out.stride(0), T, N, K, epilogue, _ptr(rt.status[1:2]))
    else:
        fn, what = L.ub_gemm_tc, "gemm_tc"
        maps = (_tmap_entry(w, 128), _tmap_entry(w2, 128) if w2 is not None else (None, 0), _tmap_entry(a, bn))
        args = (maps[0][1], maps[1][1], maps[2][1], _ptr(out),
                BF16 if out.dtype == torch.bfloat16 else F32, ldo, split_stride, T, N, K, bn, epilogue, s,
                _ptr(rt.status[1:2]))
    if key is not None:
        if len(_plans) > 8192:
            _plans.clear()
        _plans[key] = (fn, args, what, maps)     # (the maps' host memory lives as long as the plan)
    _check(fn(*args, _stream()), what)


# A product that came before with the same operands at the same places (the weights always are, the
# activations and the result because a step's scratch is handed out in the same order every time) is
# launched again from its plan: the function, its arguments and the tensor maps they point to.
_plans: dict = {}


def launch_key(a, w, out, epilogue, w2, status_ptr: int):
    """Everything a plan depends on: places, shapes and strides of the operands and of the result, the
    epilogue, and the status word the kernel reports to (another engine's tensors may come to lie at the
    same addresses with other shapes)."""
    return (a.data_ptr(), a.shape[0], a.shape[1], a.stride(0), w.data_ptr(), w.shape[0], w.stride(0), out.data_ptr(),
            out.dim(), out.shape[-1], out.stride(-2) if out.dim() > 1 else 0, out.dtype, epilogue,
            0 if w2 is None else w2.data_ptr(), status_ptr, USE_PAIRS)


def relaunch(key) -> bool:
    """Launch the product of this key from its plan; False when there is none yet."""
    plan = _plans.get(key)
    if plan is None:
        return False
    _check(plan[0](*plan[1], _stream()), plan[2])
    return True


def store_splits(T: int, N: int, K: int, n_sms: int | None = None) -> int:
    """Slices of K for a product whose result is stored (not added): worth it only with few
    tokens, where the float32 partial results are small beside the weights."""
    bn = token_tile(T, EPI_STORE)
    tiles = -(-N // 128) * -(-T // bn)
    nkb = -(-K // 64)
    slots = cta_slots(bn, EPI_STORE, n_sms)
    if T > 64 or tiles * 2 > slots or nkb < 8:
        return 1
    # the float32 partial results (written, then read) stay below a quarter of the weight bytes
    s = max(1, min(slots // tiles, nkb // 4, max(1, K // (16 * T))))
    per = -(-nkb // s)
    return -(-nkb // per)


def check_error(rt) -> None:
    rt.check_status()
