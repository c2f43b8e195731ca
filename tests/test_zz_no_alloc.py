"""The decode-attention entry point that allocates nothing (csrc/attn_noalloc.h), called
through its exported C symbol and compared with the ordinary entry point.

Some host programs may not allocate device memory once they run: they own every byte of the
GPU themselves, or an allocation would stall the streams they serve from.  For them the
library keeps the scratch of its split-key decode attention in an array of its own device
image.  This test makes two calls in a row (the array keeps what the first one wrote) and
checks both against the entry point whose scratch the caller supplies.  It is collected last
so that a run that stops at the first failure has already run every other test, and it must
pass alone in a fresh process as well as after the others.
"""
import math
from ctypes import c_float, c_int, c_longlong, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
HD = 64


def _lib():
    from ultima_b200.kernels import attn_tc
    L = attn_tc.lib(HD)                              # builds and loads the library for this head size
    fn = L.ub_attn_decode_noalloc
    fn.argtypes = [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                   c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p]
    fn.restype = c_int
    return L, fn


def _case(seed, lens, nh, nkv, ring_pages=6):
    g = torch.Generator().manual_seed(seed)
    n = len(lens)
    n_pages = n * ring_pages + 1
    table = torch.randperm(n_pages, generator=g)[:n * ring_pages].reshape(n, ring_pages).to(torch.int32).to(DEV)
    kc = (torch.randn(n_pages, nkv, 64, HD, generator=g)).to(torch.bfloat16).to(DEV)
    vc = (torch.randn(n_pages, nkv, 64, HD, generator=g)).to(torch.bfloat16).to(DEV)
    q = torch.randn(n, nh * HD, generator=g).to(torch.bfloat16).to(DEV)
    start = torch.arange(n + 1, dtype=torch.int32, device=DEV)
    before = torch.tensor([x - 1 for x in lens], dtype=torch.int32, device=DEV)
    return q, kc, vc, table, start, before


def test_no_alloc_entry_point_matches_the_ordinary_one_twice_in_a_row():
    L, noalloc = _lib()
    nh, nkv, slices = 8, 2, 3
    stream = torch.cuda.current_stream().cuda_stream
    for call, (seed, lens) in enumerate(((1, [1, 64, 200, 383]), (2, [300, 17, 129, 65]))):
        q, kc, vc, table, start, before = _case(seed, lens, nh, nkv)
        n = len(lens)
        ref = torch.full((n, nh * HD), float("nan"), dtype=torch.bfloat16, device=DEV)
        got = torch.full((n, nh * HD), float("nan"), dtype=torch.bfloat16, device=DEV)
        part_o = torch.empty(n * nh * slices * HD, dtype=torch.float32, device=DEV)
        part_ml = torch.empty(n * nh * slices * 2, dtype=torch.float32, device=DEV)
        scale = 1 / math.sqrt(HD)
        rc = L.ub_attn_mma(1, q.data_ptr(), q.stride(0), ref.data_ptr(), ref.stride(0), kc.data_ptr(), vc.data_ptr(),
                           start.data_ptr(), before.data_ptr(), table.data_ptr(), table.shape[1], table.shape[1] * 64,
                           64, n, 1, nh, nkv, 0, scale, slices, part_o.data_ptr(), part_ml.data_ptr(), stream)
        assert rc == 0
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        rc = noalloc(q.data_ptr(), q.stride(0), got.data_ptr(), got.stride(0), kc.data_ptr(), vc.data_ptr(),
                     start.data_ptr(), before.data_ptr(), table.data_ptr(), table.shape[1], table.shape[1] * 64, 64,
                     n, nh, nkv, 0, scale, slices, stream)
        assert rc == 0, f"call {call}: code {rc}"
        torch.cuda.synchronize()
        if call == 1:                                  # the first call on a device may load the module
            assert torch.cuda.mem_get_info()[0] == free_before, "the entry point changed free device memory"
        assert torch.isfinite(got.float()).all()
        err = ((got.double() - ref.double()).abs() / ref.double().abs().clamp(min=1.0)).max().item()
        assert err <= 2 ** -7, f"call {call}: error {err}"


def test_no_alloc_entry_point_refuses_what_does_not_fit():
    L, noalloc = _lib()
    q, kc, vc, table, start, before = _case(3, [10, 20], 8, 2)
    out = torch.empty(2, 8 * HD, dtype=torch.bfloat16, device=DEV)
    # 4096 sequences x 8 heads x 8 slices x 64 floats is over the 4 MiB of scratch: refused, nothing runs
    rc = noalloc(q.data_ptr(), q.stride(0), out.data_ptr(), out.stride(0), kc.data_ptr(), vc.data_ptr(),
                 start.data_ptr(), before.data_ptr(), table.data_ptr(), table.shape[1], table.shape[1] * 64, 64,
                 4096, 8, 2, 0, 0.125, 8, torch.cuda.current_stream().cuda_stream)
    assert rc == -3
