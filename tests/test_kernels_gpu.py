"""Each kernel alone against a plain PyTorch float64 restatement of the same operation, at
sizes other than the tiny models' (odd widths, head sizes in steps of 16, groups of 1, 3, 8)."""
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def _ops():
    from ultima_b200.kernels import ops
    return ops


def rel_err(got, ref):
    """Per-element error relative to max(1, |ref|), as the reference's tests measure
    (tests/unit/test_kernels_correctness.cpp:40-48)."""
    got, ref = got.double().cpu(), ref.double().cpu()
    return float(((got - ref).abs() / ref.abs().clamp(min=1.0)).max())


@pytest.mark.parametrize("table_dtype", [torch.float32, torch.bfloat16])
def test_embed(table_dtype):
    ops = _ops()
    g = torch.Generator().manual_seed(0)
    table = torch.randn(1003, 131, generator=g).to(table_dtype).to(DEV)
    ids = torch.tensor([0, 1002, 5, 5, 77], dtype=torch.int32, device=DEV)
    out = torch.empty(5, 131, dtype=torch.float32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops.embed(table, ids, out, status)
    assert torch.equal(out, table[ids.long()].float()) and int(status) == 0
    bad = torch.tensor([3, 1003], dtype=torch.int32, device=DEV)
    ops.embed(table, bad, out[:2], status)
    assert int(status) == 1 and float(out[1].abs().sum()) == 0.0


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width", [131, 896, 4100])
def test_rmsnorm(width, out_dtype):
    ops = _ops()
    g = torch.Generator().manual_seed(width)
    x = (torch.randn(7, width, generator=g) * 3).to(DEV)
    w = (1 + 0.1 * torch.randn(width, generator=g)).to(DEV)
    out = torch.empty(7, width, dtype=out_dtype, device=DEV)
    ops.rmsnorm(x, w, out, 1e-5)
    xd = x.double()
    ref = xd * w.double() / torch.sqrt((xd * xd).mean(-1, keepdim=True) + 1e-5)
    assert rel_err(out, ref) <= (2e-6 if out_dtype == torch.float32 else 2 ** -8)
    rows = torch.tensor([6, 0, 3], dtype=torch.int32, device=DEV)
    out2 = torch.empty(3, width, dtype=out_dtype, device=DEV)
    ops.rmsnorm(x, w, out2, 1e-5, rows)
    assert torch.equal(out2, out[rows.long()])


@pytest.mark.parametrize("dt", [(torch.float32, torch.float32, torch.float32),
                                (torch.bfloat16, torch.bfloat16, torch.bfloat16),
                                (torch.bfloat16, torch.float32, torch.float32),
                                (torch.bfloat16, torch.bfloat16, torch.float32)])
@pytest.mark.parametrize("shape", [(1, 517, 131), (5, 64, 200), (70, 333, 129), (130, 96, 1000)])
def test_gemm_simt(shape, dt):
    ops = _ops()
    M, K, N = shape
    ta, tw, to = dt
    g = torch.Generator().manual_seed(M * 7 + N)
    a = torch.randn(M, K, generator=g).to(ta).to(DEV)
    w = (torch.randn(N, K, generator=g) * 0.05).to(tw).to(DEV)
    w2 = (torch.randn(N, K, generator=g) * 0.05).to(tw).to(DEV)
    ref = a.double() @ w.double().T
    out = torch.empty(M, N, dtype=to, device=DEV)
    ops.gemm_simt(a, w, out)
    tol = 1e-5 if to == torch.float32 else 2 ** -8
    assert rel_err(out, ref) <= tol
    if to == torch.float32:
        acc = torch.randn(M, N, generator=g).to(DEV)
        before = acc.clone()
        ops.gemm_simt(a, w, acc, ops.EPI_ADD)
        assert rel_err(acc, before.double() + ref) <= 1e-5
    ref2 = a.double() @ w2.double().T
    ops.gemm_simt(a, w, out, ops.EPI_SWIGLU, w2=w2)
    assert rel_err(out, ref / (1 + torch.exp(-ref)) * ref2) <= tol
    # a view with a row stride (columns of a wider matrix), as the q part of [q | k | v]
    wide = torch.randn(M, K + 24, generator=g).to(ta).to(DEV)
    ops.gemm_simt(wide[:, 8:8 + K], w, out)
    assert rel_err(out, wide[:, 8:8 + K].double() @ w.double().T) <= tol


def _paged(n_seqs, lens, nkv, hd, dtype, ring_pages, seed, page=64):
    """Random K, V for sequences of the given lengths, stored in shuffled pages (ring_pages
    pages a sequence, wrapped).  Returns caches, table and the dense tensors."""
    g = torch.Generator().manual_seed(seed)
    n_pages = n_seqs * ring_pages + 3
    perm = torch.randperm(n_pages, generator=g)[:n_seqs * ring_pages].reshape(n_seqs, ring_pages)
    kc = torch.full((n_pages, nkv, page, hd), float("nan"), dtype=dtype)
    vc = torch.full((n_pages, nkv, page, hd), float("nan"), dtype=dtype)
    dense = []
    for s, n in enumerate(lens):
        k = torch.randn(n, nkv, hd, generator=g).to(dtype)
        v = torch.randn(n, nkv, hd, generator=g).to(dtype)
        dense.append((k, v))
        for p in range(n):
            li = p % (ring_pages * page)
            kc[perm[s, li // page], :, li % page] = k[p]
            vc[perm[s, li // page], :, li % page] = v[p]
    return kc.to(DEV), vc.to(DEV), perm.to(torch.int32).to(DEV), dense


def _attn_ref(q, k, v, pos, window, scale):
    """q [nh, hd] at position pos over k, v [n, nkv, hd] (float64)."""
    nh, nkv = q.shape[0], k.shape[1]
    lo = max(0, pos + 1 - window) if window else 0
    out = torch.zeros_like(q)
    for h in range(nh):
        g = h // (nh // nkv)
        s = (k[lo:pos + 1, g] @ q[h]) * scale
        out[h] = torch.softmax(s, 0) @ v[lo:pos + 1, g]
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("cfg", [dict(nh=6, nkv=2, hd=48, window=0), dict(nh=8, nkv=1, hd=16, window=0),
                                 dict(nh=4, nkv=4, hd=80, window=37), dict(nh=3, nkv=3, hd=256, window=0)])
def test_attn_simple(cfg, dtype):
    ops = _ops()
    nh, nkv, hd, window = cfg["nh"], cfg["nkv"], cfg["hd"], cfg["window"]
    lens = [1, 70, 129, 600]
    ring_pages = 10
    kc, vc, table, dense = _paged(len(lens), lens, nkv, hd, dtype, ring_pages, seed=hd)
    # queries: for each sequence its last token and, for longer ones, two earlier tokens
    toks = [(s, p) for s, n in enumerate(lens) for p in sorted({n - 1, n // 2, 0})]
    g = torch.Generator().manual_seed(1)
    q = torch.randn(len(toks), nh * hd + 8, generator=g).to(dtype).to(DEV)[:, :nh * hd]   # strided rows
    out = torch.empty(len(toks), nh * hd, dtype=dtype, device=DEV)
    pos = torch.tensor([p for _, p in toks], dtype=torch.int32, device=DEV)
    seq = torch.tensor([s for s, _ in toks], dtype=torch.int32, device=DEV)
    scale = 1 / math.sqrt(hd)
    ops.attn_simple(q, kc, vc, out, pos, seq, table, ring_pages * 64, 64, nh, nkv, hd, window, scale)
    for i, (s, p) in enumerate(toks):
        k, v = dense[s]
        ref = _attn_ref(q[i].double().cpu().view(nh, hd), k.double(), v.double(), p, window, scale)
        err = rel_err(out[i].view(nh, hd), ref)
        assert err <= (2e-5 if dtype == torch.float32 else 2 ** -7), (i, s, p, err)


def test_attention_finds_a_far_key_and_respects_the_window_edge():
    """One key among hundreds is made to stand out; with a window that just excludes it the
    output must not see it, with one position more it must."""
    ops = _ops()
    nh, nkv, hd, n = 2, 1, 32, 700
    g = torch.Generator().manual_seed(3)
    k = torch.randn(n, nkv, hd, generator=g) * 0.1
    v = torch.randn(n, nkv, hd, generator=g) * 0.1
    q = torch.randn(1, nh * hd, generator=g) * 0.1
    far = 213
    k[far, 0] = q[0, :hd] * 400.0            # a huge score for head 0 at position 213
    v[far, 0] = 5.0
    ring_pages = 11
    kc = torch.full((ring_pages, nkv, 64, hd), float("nan"))
    vc = torch.full((ring_pages, nkv, 64, hd), float("nan"))
    for p in range(n):
        kc[p // 64, :, p % 64], vc[p // 64, :, p % 64] = k[p], v[p]
    table = torch.arange(ring_pages, dtype=torch.int32).view(1, -1).to(DEV)
    pos = torch.tensor([n - 1], dtype=torch.int32, device=DEV)
    seq = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = torch.empty(1, nh * hd, device=DEV)
    args = (q.to(DEV), kc.to(DEV), vc.to(DEV), out, pos, seq, table, ring_pages * 64, 64, nh, nkv, hd)
    ops.attn_simple(*args, 0, 1 / math.sqrt(hd))
    assert float(out[0, :hd].min()) > 4.9                      # head 0 is all that one value
    ops.attn_simple(*args, n - 1 - far, 1 / math.sqrt(hd))     # window ends one short of it
    assert float(out[0, :hd].abs().max()) < 1.0
    ops.attn_simple(*args, n - far, 1 / math.sqrt(hd))         # window just reaches it
    assert float(out[0, :hd].min()) > 4.9


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("cfg", [dict(nh=6, nkv=2, hd=48), dict(nh=8, nkv=1, hd=16), dict(nh=2, nkv=2, hd=112),
                                 dict(nh=4, nkv=2, hd=128), dict(nh=3, nkv=1, hd=64), dict(nh=2, nkv=1, hd=256)])
def test_qk_prepare_norm_rotation_and_cache_write(cfg, dtype):
    ops = _ops()
    nh, nkv, hd = cfg["nh"], cfg["nkv"], cfg["hd"]
    half, eps, theta = hd // 2, 1e-5, 1e4
    toks = [(0, 0), (0, 1), (1, 63), (1, 64), (2, 150), (2, 151)]          # (sequence, position)
    T = len(toks)
    g = torch.Generator().manual_seed(hd)
    qkv = torch.randn(T, (nh + 2 * nkv) * hd, generator=g).to(dtype)
    qw, kw = 1 + 0.1 * torch.randn(hd, generator=g), 1 + 0.1 * torch.randn(hd, generator=g)
    inv = 1.0 / theta ** (2.0 * torch.arange(half, dtype=torch.float64) / hd)
    ang = torch.arange(200, dtype=torch.float64)[:, None] * inv[None]
    cos, sin = torch.cos(ang).float(), torch.sin(ang).float()
    ring_pages, n_pages = 2, 8                                             # ring of 128 positions
    table = torch.tensor([[5, 1], [0, 7], [3, 2]], dtype=torch.int32)
    kc = torch.zeros(n_pages, nkv, 64, hd, dtype=dtype, device=DEV)
    vc = torch.zeros(n_pages, nkv, 64, hd, dtype=dtype, device=DEV)
    dev_qkv = qkv.clone().to(DEV)
    ops.qk_prepare(dev_qkv, qw.to(DEV), kw.to(DEV), cos.to(DEV), sin.to(DEV),
                   torch.tensor([p for _, p in toks], dtype=torch.int32, device=DEV),
                   torch.tensor([s for s, _ in toks], dtype=torch.int32, device=DEV),
                   kc, vc, table.to(DEV), ring_pages * 64, 64, nh, nkv, hd, eps)

    def prep(x, w, p):          # x [heads, hd] float64
        x = x * w.double() / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
        a, b = x[:, :half], x[:, half:]
        c, s = torch.cos(ang[p])[None], torch.sin(ang[p])[None]
        return torch.cat([a * c - b * s, a * s + b * c], -1)
    tol = 1e-5 if dtype == torch.float32 else 2 ** -7
    for t, (s, p) in enumerate(toks):
        row = qkv[t].double()
        q_ref = prep(row[:nh * hd].view(nh, hd), qw, p)
        k_ref = prep(row[nh * hd:(nh + nkv) * hd].view(nkv, hd), kw, p)
        v_ref = row[(nh + nkv) * hd:].view(nkv, hd)
        assert rel_err(dev_qkv[t, :nh * hd].view(nh, hd), q_ref) <= tol
        li = p % (ring_pages * 64)
        pg = int(table[s, li // 64])
        assert rel_err(kc[pg, :, li % 64], k_ref) <= tol, (t, s, p)
        assert rel_err(vc[pg, :, li % 64], v_ref) <= (0 if dtype == torch.float32 else tol)
    # a run that reads another run's cache writes nothing
    kc2, vc2 = torch.zeros_like(kc), torch.zeros_like(vc)
    ops.qk_prepare(qkv.clone().to(DEV), qw.to(DEV), kw.to(DEV), cos.to(DEV), sin.to(DEV),
                   torch.tensor([p for _, p in toks], dtype=torch.int32, device=DEV),
                   torch.tensor([s for s, _ in toks], dtype=torch.int32, device=DEV),
                   kc2, vc2, table.to(DEV), ring_pages * 64, 64, nh, nkv, hd, eps, write_kv=False)
    assert float(kc2.abs().sum()) == 0 and float(vc2.abs().sum()) == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("cfg", [dict(nh=4, nkv=2, hd=128, norm=True, rot=True), dict(nh=5, nkv=1, hd=64, norm=True, rot=True),
                                 dict(nh=2, nkv=1, hd=256, norm=False, rot=True), dict(nh=3, nkv=3, hd=128, norm=True, rot=False),
                                 dict(nh=3, nkv=1, hd=80, norm=True, rot=True)])
def test_qk_prepare_for_prompts(cfg, dtype):
    """Hundreds of tokens of two sequences (a block a token, its warps walking over the heads),
    with and without norm and rotation, q written to a matrix of its own."""
    ops = _ops()
    nh, nkv, hd = cfg["nh"], cfg["nkv"], cfg["hd"]
    half, eps, theta = hd // 2, 1e-5, 1e4
    lens = [190, 141]
    toks = [(s, p) for s, n in enumerate(lens) for p in range(n)]
    T = len(toks)
    g = torch.Generator().manual_seed(hd + nh)
    qkv = torch.randn(T, (nh + 2 * nkv) * hd, generator=g).to(dtype)
    qw = (1 + 0.1 * torch.randn(hd, generator=g)) if cfg["norm"] else None
    kw = (1 + 0.1 * torch.randn(hd, generator=g)) if cfg["norm"] else None
    inv = 1.0 / theta ** (2.0 * torch.arange(half, dtype=torch.float64) / hd)
    ang = torch.arange(256, dtype=torch.float64)[:, None] * inv[None]
    cos = torch.cos(ang).float().to(DEV) if cfg["rot"] else None
    sin = torch.sin(ang).float().to(DEV) if cfg["rot"] else None
    n_pages = 9
    table = torch.tensor([[5, 1, 8], [0, 7, 3]], dtype=torch.int32)
    kc = torch.zeros(n_pages, nkv, 64, hd, dtype=dtype, device=DEV)
    vc = torch.zeros(n_pages, nkv, 64, hd, dtype=dtype, device=DEV)
    q_out = torch.full((T, nh * hd), float("nan"), dtype=dtype, device=DEV)
    ops.qk_prepare(qkv.to(DEV), None if qw is None else qw.to(DEV), None if kw is None else kw.to(DEV), cos, sin,
                   torch.tensor([p for _, p in toks], dtype=torch.int32, device=DEV),
                   torch.tensor([s for s, _ in toks], dtype=torch.int32, device=DEV),
                   kc, vc, table.to(DEV), 3 * 64, 64, nh, nkv, hd, eps, q_out=q_out)

    def prep(x, w, p):          # x [T, heads, hd] float64, p [T]
        if w is not None:
            x = x * w.double() / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
        if not cfg["rot"]:
            return x
        a, b = x[..., :half], x[..., half:]
        c, s = torch.cos(ang[p])[:, None], torch.sin(ang[p])[:, None]
        return torch.cat([a * c - b * s, a * s + b * c], -1)
    pos = torch.tensor([p for _, p in toks])
    rows = qkv.double()
    tol = 1e-5 if dtype == torch.float32 else 2 ** -7
    q_ref = prep(rows[:, :nh * hd].view(T, nh, hd), qw, pos)
    k_ref = prep(rows[:, nh * hd:(nh + nkv) * hd].view(T, nkv, hd), kw, pos)
    v_ref = rows[:, (nh + nkv) * hd:].view(T, nkv, hd)
    assert rel_err(q_out.view(T, nh, hd), q_ref) <= tol
    for t, (s, p) in enumerate(toks):
        pg = int(table[s, p // 64])
        assert rel_err(kc[pg, :, p % 64], k_ref[t]) <= tol, (t, s, p)
        assert rel_err(vc[pg, :, p % 64], v_ref[t]) <= (0 if dtype == torch.float32 else tol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("cfg", [dict(nh=4, nkv=2, hd=128, rd=64, inter=False), dict(nh=3, nkv=1, hd=64, rd=64, inter=True),
                                 dict(nh=5, nkv=5, hd=48, rd=20, inter=True), dict(nh=2, nkv=1, hd=256, rd=96, inter=False),
                                 dict(nh=2, nkv=2, hd=16, rd=2, inter=False)])
def test_qk_prepare_rotates_part_of_a_head_and_interleaved_pairs(cfg, dtype):
    """The first ``rd`` columns of a head rotated in pairs (j, j + rd/2) or (2j, 2j + 1), the rest passing
    through (normed all the same); and the dense route: keys and values to matrices of their own instead
    of the cache, then ``kv_write`` into the pages, which must give the cache the direct route gives."""
    ops = _ops()
    nh, nkv, hd, rd, inter = cfg["nh"], cfg["nkv"], cfg["hd"], cfg["rd"], cfg["inter"]
    eps, theta, rhalf = 1e-5, 1e4, cfg["rd"] // 2
    toks = [(0, 0), (0, 1), (1, 63), (1, 64), (2, 150), (2, 151), (2, 152)]
    T = len(toks)
    g = torch.Generator().manual_seed(hd + rd)
    qkv = torch.randn(T, (nh + 2 * nkv) * hd, generator=g).to(dtype)
    qw, kw = 1 + 0.1 * torch.randn(hd, generator=g), 1 + 0.1 * torch.randn(hd, generator=g)
    ang = torch.arange(200, dtype=torch.float64)[:, None] / theta ** (2.0 * torch.arange(rhalf, dtype=torch.float64) / rd)[None]
    cos, sin = torch.cos(ang).float().to(DEV), torch.sin(ang).float().to(DEV)
    table = torch.tensor([[5, 1, 6], [0, 7, 4], [3, 2, 8]], dtype=torch.int32, device=DEV)
    pos = torch.tensor([p for _, p in toks], dtype=torch.int32, device=DEV)
    seq = torch.tensor([s for s, _ in toks], dtype=torch.int32, device=DEV)

    def prep(x, w, p):          # x [heads, hd] float64
        x = x * w.double() / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
        c, s_ = torch.cos(ang[p])[None], torch.sin(ang[p])[None]
        y = x.clone()
        if inter:
            a, b = x[:, 0:rd:2], x[:, 1:rd:2]
            y[:, 0:rd:2], y[:, 1:rd:2] = a * c - b * s_, a * s_ + b * c
        else:
            a, b = x[:, :rhalf], x[:, rhalf:rd]
            y[:, :rhalf], y[:, rhalf:rd] = a * c - b * s_, a * s_ + b * c
        return y
    kc = torch.zeros(9, nkv, 64, hd, dtype=dtype, device=DEV)
    vc = torch.zeros_like(kc)
    q = torch.full((T, nh * hd), float("nan"), dtype=dtype, device=DEV)
    ops.qk_prepare(qkv.to(DEV), qw.to(DEV), kw.to(DEV), cos, sin, pos, seq, kc, vc, table, 192, 64, nh, nkv, hd, eps,
                   q_out=q, rotary_dim=rd, interleaved=inter)
    tol = 1e-5 if dtype == torch.float32 else 2 ** -7
    for t, (s_i, p) in enumerate(toks):
        row = qkv[t].double()
        assert rel_err(q[t].view(nh, hd), prep(row[:nh * hd].view(nh, hd), qw, p)) <= tol, (cfg, t)
        pg = int(table[s_i, p // 64])
        assert rel_err(kc[pg, :, p % 64], prep(row[nh * hd:(nh + nkv) * hd].view(nkv, hd), kw, p)) <= tol, (cfg, t)
        assert rel_err(vc[pg, :, p % 64], row[(nh + nkv) * hd:].view(nkv, hd)) <= (0 if dtype == torch.float32 else tol)
    # the dense route: norm here, rotation by a call of its own, then the write into the pages
    kc2, vc2 = torch.zeros_like(kc), torch.zeros_like(vc)
    q2 = torch.full((T, nh * hd), float("nan"), dtype=dtype, device=DEV)
    kbuf = torch.full((2, T, nkv * hd), float("nan"), dtype=dtype, device=DEV)
    ops.qk_prepare(qkv.to(DEV), qw.to(DEV), kw.to(DEV), None, None, pos, seq, kc2, vc2, table, 192, 64, nh, nkv, hd, eps,
                   q_out=q2, kv_out=(kbuf[0], kbuf[1]))
    assert float(kc2.abs().sum()) == 0 and float(vc2.abs().sum()) == 0           # nothing went into the cache yet
    ops.rotate_pairs(q2.view(T, nh, hd), cos, sin, pos, rd, inter)
    ops.rotate_pairs(kbuf[0].view(T, nkv, hd), cos, sin, pos, rd, inter)
    ops.kv_write(kbuf[0], kbuf[1], pos, seq, kc2, vc2, table, 192, 64, nkv, hd)
    two = 2e-6 if dtype == torch.float32 else 2 ** -6            # bfloat16: rounded once more between norm and rotation
    assert rel_err(q2, q.double()) <= two and rel_err(kc2, kc.double()) <= two
    assert torch.equal(vc2, vc)
    with pytest.raises(ops.KernelError, match="rotary size"):
        ops.qk_prepare(qkv.to(DEV), qw.to(DEV), kw.to(DEV), cos, sin, pos, seq, kc, vc, table, 192, 64, nh, nkv, hd, eps,
                       q_out=q, rotary_dim=hd + 2)


def test_fill_normal_is_the_host_generator_bit_for_bit():
    """The fill kernel against the tests' own copy of the counter-based generator (tests/plain_random.py):
    the same bits in float32, and the same after rounding to bfloat16."""
    import plain_random as R
    ops = _ops()
    n = 300000
    for key, shift, std in ((R.tensor_key(7, "model.embed_tokens.weight"), 0.0, 0.02), (12345, 1.0, 0.05), ((1 << 63) - 1, 0.0, 1.0)):
        want = (np.float32(shift) + np.float32(std) * R.normal_array(key, n)).astype(np.float32)
        got = torch.empty(n, device=DEV)
        ops.fill_normal(got, key, shift, std)
        assert np.array_equal(got.cpu().numpy().view(np.uint32), want.view(np.uint32)), key
        got16 = torch.empty(n, dtype=torch.bfloat16, device=DEV)
        ops.fill_normal(got16, key, shift, std)
        assert np.array_equal(got16.view(torch.int16).cpu().numpy().view(np.uint16), R.to_bfloat16_bits(want)), key


def test_models_drawn_on_the_device_and_on_the_host_are_the_same_model():
    import ultima_b200 as u
    from conftest import TINY
    from ultima_b200.weights import random_tensors, random_tensors_on_device
    cfg = u.config_from_dict(TINY["E"])
    specs = u.model_spec_for(cfg).weight_specs()
    for run_dtype in (torch.bfloat16, torch.float32):
        dev = random_tensors_on_device(specs, 5, run_dtype, DEV)
        host = random_tensors(specs, 5, run_dtype)
        for s_ in specs:
            d, h = dev[s_.name].cpu(), host[s_.name]
            if s_.kind == "vector":                                # held in 32-bit on the device on both paths
                h = random_tensors([s_], 5, torch.float32)[s_.name]
            assert d.dtype == h.dtype and torch.equal(d, h), (s_.name, run_dtype)


def test_silu_mul_convert_add_fill():
    ops = _ops()
    g = torch.Generator().manual_seed(9)
    gu = torch.randn(5, 2 * 177, generator=g).to(DEV)
    out = torch.empty(5, 177, device=DEV)
    ops.silu_mul(gu, out)
    gd = gu.double()
    assert rel_err(out, gd[:, :177] / (1 + torch.exp(-gd[:, :177])) * gd[:, 177:]) <= 1e-6
    b = torch.empty(5, 2 * 177, dtype=torch.bfloat16, device=DEV)
    ops.convert(gu, b)
    assert torch.equal(b, gu.to(torch.bfloat16))
    acc = torch.ones(5, 2 * 177, device=DEV)
    ops.add_into(acc, b)
    assert torch.equal(acc, 1 + b.float())
    big = torch.empty(1 << 20, device=DEV)
    ops.fill_normal(big, 1234, 1.0, 0.05)
    assert abs(float(big.mean()) - 1.0) < 1e-3 and abs(float(big.std()) - 0.05) < 1e-3
    again = torch.empty(1 << 20, device=DEV)
    ops.fill_normal(again, 1234, 1.0, 0.05)
    assert torch.equal(big, again)


# ---------------------------------------------------------------------------------------
# the tensor-core product against the CUDA-core product and float64
# ---------------------------------------------------------------------------------------
def _tc():
    from ultima_b200.kernels import gemm_tc
    from ultima_b200.engine import Runtime
    return gemm_tc, Runtime(DEV, torch.bfloat16)


@pytest.mark.parametrize("shape", [(1, 64, 128), (5, 96, 200), (16, 512, 128), (33, 1024, 384), (64, 4096, 256),
                                   (130, 320, 96), (300, 200, 1000), (513, 2048, 640)])
def test_gemm_tc_store(shape):
    gemm_tc, rt = _tc()
    ops = _ops()
    T, K, N = shape
    g = torch.Generator().manual_seed(T + K)
    a = torch.randn(T, K, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    ref = a.double() @ w.double().T
    for dt in (torch.bfloat16, torch.float32):
        out = torch.full((T, N), float("nan"), dtype=dt, device=DEV)
        assert gemm_tc.accepts(a, w, out, ops.EPI_STORE, None)
        gemm_tc.gemm(a, w, out, ops.EPI_STORE, None, rt)
        torch.cuda.synchronize()
        gemm_tc.check_error(rt)
        # the tensor cores align and truncate the products of one instruction: the error grows with K
        assert rel_err(out, ref) <= (2 ** -8 if dt == torch.bfloat16 else max(2e-6, K * 2.0 ** -25)), (shape, dt)


def test_product_plans_follow_shapes_and_contents():
    """The runtime launches a product again from a remembered plan when operands and result lie where they
    lay before.  Other shapes at the same addresses get a plan of their own, other contents at the same
    addresses go through the old plan and give the new result, and a second runtime reports to its own
    status word."""
    gemm_tc, rt = _tc()
    rt2 = _tc()[1]
    ops = _ops()
    g = torch.Generator().manual_seed(77)
    abuf = torch.empty(1 << 20, dtype=torch.bfloat16, device=DEV)
    wbuf = torch.empty(1 << 20, dtype=torch.bfloat16, device=DEV)
    obuf = torch.empty(1 << 20, dtype=torch.float32, device=DEV)
    seen = set()
    for rep, (T, K, N) in enumerate([(8, 512, 256), (8, 512, 256), (16, 256, 256), (8, 256, 512), (8, 512, 256)]):
        a = abuf[:T * K].view(T, K)
        w = wbuf[:N * K].view(N, K)
        out = obuf[:T * N].view(T, N)
        a.copy_(torch.randn(T, K, generator=g).to(torch.bfloat16))
        w.copy_((torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16))
        out.fill_(float("nan"))
        for r in (rt, rt2):
            key = gemm_tc.launch_key(a, w, out, ops.EPI_STORE, None, r._status_ptr)
            known = key in gemm_tc._plans
            r.matmul(a, w, out, ops.EPI_STORE)
            torch.cuda.synchronize()
            gemm_tc.check_error(r)
            assert key in gemm_tc._plans
            assert rel_err(out, a.double() @ w.double().T) <= max(2e-6, K * 2.0 ** -25), (rep, T, K, N, known)
            seen.add(key)
    assert len(seen) == 6          # three shapes, two runtimes: the repeats found their plans


@pytest.mark.parametrize("shape", [(3, 4096, 512, None), (8, 12288, 256, None), (64, 2048, 128, 4), (200, 1024, 300, 2),
                                   (7, 960, 130, 3)])
def test_gemm_tc_add_with_and_without_k_split(shape):
    gemm_tc, rt = _tc()
    ops = _ops()
    T, K, N, splits = shape
    g = torch.Generator().manual_seed(K)
    a = torch.randn(T, K, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    acc = torch.randn(T, N, generator=g).to(DEV)
    ref = acc.double() + a.double() @ w.double().T
    gemm_tc.gemm(a, w, acc, ops.EPI_ADD, None, rt, splits=splits)
    torch.cuda.synchronize()
    gemm_tc.check_error(rt)
    assert rel_err(acc, ref) <= max(2e-6, K * 2.0 ** -25), shape


@pytest.mark.parametrize("shape", [(2, 64, 192), (40, 96, 320), (128, 4096, 384), (257, 512, 130)])
def test_gemm_tc_gate_product(shape):
    gemm_tc, rt = _tc()
    ops = _ops()
    T, K, F = shape
    g = torch.Generator().manual_seed(F)
    a = torch.randn(T, K, generator=g).to(torch.bfloat16).to(DEV)
    wgu = (torch.randn(2 * F, K, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    out = torch.full((T, F), float("nan"), dtype=torch.bfloat16, device=DEV)
    gemm_tc.gemm(a, wgu[:F], out, ops.EPI_SWIGLU, wgu[F:], rt)
    torch.cuda.synchronize()
    gemm_tc.check_error(rt)
    gt, up = a.double() @ wgu[:F].double().T, a.double() @ wgu[F:].double().T
    assert rel_err(out, gt / (1 + torch.exp(-gt)) * up) <= 2 ** -8, shape


def test_gemm_tc_views_and_what_it_refuses():
    gemm_tc, rt = _tc()
    ops = _ops()
    g = torch.Generator().manual_seed(0)
    wide = torch.randn(50, 256 + 64, generator=g).to(torch.bfloat16).to(DEV)
    a = wide[:, 64:]                                   # rows start on 16-byte boundaries: taken
    w = (torch.randn(96, 256, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    out = torch.empty(50, 96, dtype=torch.float32, device=DEV)
    assert gemm_tc.accepts(a, w, out, ops.EPI_STORE, None)
    gemm_tc.gemm(a, w, out, ops.EPI_STORE, None, rt)
    assert rel_err(out, a.double() @ w.double().T) <= 2e-5
    assert not gemm_tc.accepts(wide[:, 3:259], w, out, ops.EPI_STORE, None)          # misaligned rows
    assert not gemm_tc.accepts(a[:, :100], w[:, :100], out, ops.EPI_STORE, None)     # K not a multiple of 8
    assert not gemm_tc.accepts(a.float(), w, out, ops.EPI_STORE, None)
    # the runtime sends refused shapes to the CUDA-core kernel and gets the same answer
    a2, w2 = a[:, :100].contiguous(), w[:, :100].contiguous()
    rt.matmul(a2, w2, out)
    assert rel_err(out, a2.double() @ w2.double().T) <= 2e-5


# ---------------------------------------------------------------------------------------
# tensor-core attention against the float64 restatement
# ---------------------------------------------------------------------------------------
class _KV:
    def __init__(self, k, v, table, ring, window):
        self.k, self.v, self.table, self.ring, self.page, self.window = k, v, table, ring, 64, window


class _B:
    pass


def _attn_tc_case(nh, nkv, hd, window, befores, news, seed, slices=None, ring_pages=12, kernel=None):
    """Sequences with ``befores[i]`` cached positions bring ``news[i]`` new tokens."""
    from ultima_b200.kernels import attn_tc
    from ultima_b200.engine import Runtime
    rt = Runtime(DEV, torch.bfloat16)
    lens = [b + n for b, n in zip(befores, news)]
    kc, vc, table, dense = _paged(len(lens), lens, nkv, hd, torch.bfloat16, ring_pages, seed)
    T = sum(news)
    g = torch.Generator().manual_seed(seed + 1)
    qkv = torch.randn(T, (nh + 2 * nkv) * hd, generator=g).to(torch.bfloat16).to(DEV)
    q = qkv[:, :nh * hd]
    out = torch.full((T, nh * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
    b = _B()
    start = [0]
    for n in news:
        start.append(start[-1] + n)
    b.seq_start = torch.tensor(start, dtype=torch.int32, device=DEV)
    b.seq_before = torch.tensor(befores, dtype=torch.int32, device=DEV)
    b.n_seqs, b.max_new, b.max_after = len(lens), max(news), max(lens)
    kv = _KV(kc, vc, table, ring_pages * 64, window or None)
    assert attn_tc.accepts(q, kv, hd, nh, nkv)
    attn_tc.attention(q, kv, out, b, nh, nkv, hd, 1 / math.sqrt(hd), rt, slices=slices, kernel=kernel)
    torch.cuda.synchronize()
    rt.check_status()
    worst = 0.0
    for s, (bf, n) in enumerate(zip(befores, news)):
        k, v = dense[s]
        for t in range(n):
            ref = _attn_ref(q[start[s] + t].double().cpu().view(nh, hd), k.double(), v.double(), bf + t, window, 1 / math.sqrt(hd))
            got = out[start[s] + t].view(nh, hd)
            assert torch.isfinite(got).all(), (s, t)
            worst = max(worst, rel_err(got, ref))
    return worst


@pytest.mark.parametrize("cfg", [dict(nh=8, nkv=2, hd=128, window=0), dict(nh=6, nkv=3, hd=48, window=0),
                                 dict(nh=8, nkv=1, hd=32, window=0), dict(nh=4, nkv=2, hd=16, window=0),
                                 dict(nh=6, nkv=2, hd=80, window=50), dict(nh=2, nkv=2, hd=256, window=0),
                                 dict(nh=5, nkv=5, hd=64, window=130)])
def test_attn_mma_prefill(cfg):
    # whole prompts of unequal lengths, and continued prompts (cached positions before the new ones)
    for befores, news in (([0, 0, 0, 0], [1, 17, 64, 200]), ([5, 64, 130, 0], [70, 1, 33, 129])):
        err = _attn_tc_case(cfg["nh"], cfg["nkv"], cfg["hd"], cfg["window"], befores, news, seed=cfg["hd"], kernel="mma")
        assert err <= 2 ** -7, (cfg, befores, news, err)


@pytest.mark.parametrize("cfg", [dict(nh=8, nkv=2, hd=128, window=0), dict(nh=8, nkv=1, hd=64, window=0),
                                 dict(nh=4, nkv=4, hd=128, window=0), dict(nh=4, nkv=2, hd=64, window=50),
                                 dict(nh=32, nkv=2, hd=128, window=0), dict(nh=2, nkv=1, hd=128, window=130),
                                 dict(nh=10, nkv=2, hd=128, window=0), dict(nh=6, nkv=2, hd=64, window=0),
                                 dict(nh=7, nkv=1, hd=64, window=33)])
@pytest.mark.parametrize("wide", [0, 2])
def test_attn_tcgen05_prefill(cfg, wide):
    """The tcgen05 prefill kernels (128 and 256 rows a CTA): scores and output in tensor memory."""
    from ultima_b200.kernels import attn_tc
    assert attn_tc.tcgen05_fits(cfg["hd"], cfg["nh"], cfg["nkv"])
    was = attn_tc.WIDE
    attn_tc.set_wide(wide)
    try:
        for befores, news in (([0, 0, 0, 0], [1, 17, 64, 200]), ([5, 64, 130, 0], [70, 1, 33, 129]), ([0], [700])):
            err = _attn_tc_case(cfg["nh"], cfg["nkv"], cfg["hd"], cfg["window"], befores, news, seed=cfg["hd"] + 3)
            assert err <= 2 ** -7, (cfg, befores, news, err)
    finally:
        attn_tc.set_wide(was)


@pytest.mark.parametrize("cfg", [dict(nh=8, nkv=2, hd=128, window=0), dict(nh=8, nkv=1, hd=64, window=0),
                                 dict(nh=16, nkv=1, hd=128, window=0), dict(nh=4, nkv=2, hd=64, window=50)])
@pytest.mark.parametrize("slices", [None, 1, 3])
def test_attn_tcgen05_decode(cfg, slices):
    befores = [0, 63, 64, 300, 700]
    err = _attn_tc_case(cfg["nh"], cfg["nkv"], cfg["hd"], cfg["window"], befores, [1] * 5, seed=cfg["hd"] + 9,
                        slices=slices, kernel="tc")
    assert err <= 2 ** -7, (cfg, slices, err)


@pytest.mark.parametrize("wide", [0, 2])
def test_attn_tcgen05_rescales_when_the_maximum_grows(wide):
    """Keys whose scores grow along the sequence force the reference maximum up again and again."""
    from ultima_b200.kernels import attn_tc
    from ultima_b200.engine import Runtime
    was = attn_tc.WIDE
    attn_tc.set_wide(wide)
    rt = Runtime(DEV, torch.bfloat16)
    nh = nkv = 1
    hd, n = 128, 400
    g = torch.Generator().manual_seed(0)
    qrow = torch.randn(hd, generator=g)
    qrow = qrow / qrow.norm()
    k = torch.randn(n, 1, hd, generator=g) * 0.1
    k[:, 0] += qrow[None] * torch.linspace(0, 300, n)[:, None]          # scores rise by ~26 log2 units a page
    v = torch.randn(n, 1, hd, generator=g)
    q = (qrow[None].repeat(n, 1) * math.sqrt(hd)).to(torch.bfloat16).to(DEV)
    pages = 7
    kc = torch.full((pages, 1, 64, hd), float("nan"), dtype=torch.bfloat16)
    vc = torch.full((pages, 1, 64, hd), float("nan"), dtype=torch.bfloat16)
    for p_ in range(n):
        kc[p_ // 64, 0, p_ % 64], vc[p_ // 64, 0, p_ % 64] = k[p_, 0].to(torch.bfloat16), v[p_, 0].to(torch.bfloat16)
    b = _B()
    b.seq_start = torch.tensor([0, n], dtype=torch.int32, device=DEV)
    b.seq_before = torch.tensor([0], dtype=torch.int32, device=DEV)
    b.n_seqs, b.max_new, b.max_after = 1, n, n
    kv = _KV(kc.to(DEV), vc.to(DEV), torch.arange(pages, dtype=torch.int32).view(1, -1).to(DEV), pages * 64, None)
    out = torch.full((n, hd), float("nan"), dtype=torch.bfloat16, device=DEV)
    attn_tc.attention(q, kv, out, b, nh, nkv, hd, 1 / math.sqrt(hd), rt)
    torch.cuda.synchronize()
    rt.check_status()
    kd, vd = kc[:, 0].reshape(-1, hd)[:n].double(), vc[:, 0].reshape(-1, hd)[:n].double()
    attn_tc.set_wide(was)
    for t in (0, 63, 64, 200, 399):
        s = (kd[:t + 1] @ q[t].double().cpu()) / math.sqrt(hd)
        ref = torch.softmax(s, 0) @ vd[:t + 1]
        assert rel_err(out[t], ref) <= 2 ** -6, t


@pytest.mark.parametrize("cfg", [dict(nh=8, nkv=2, hd=128, window=0), dict(nh=6, nkv=3, hd=48, window=0),
                                 dict(nh=8, nkv=1, hd=32, window=0), dict(nh=16, nkv=1, hd=16, window=0),
                                 dict(nh=6, nkv=2, hd=80, window=50), dict(nh=2, nkv=2, hd=256, window=0),
                                 dict(nh=32, nkv=1, hd=64, window=0)])
@pytest.mark.parametrize("slices", [None, 1, 3])
def test_attn_mma_decode(cfg, slices):
    # one token a sequence, at unequal lengths: position 0, a page edge, mid page, many pages
    befores = [0, 63, 64, 300, 700]
    err = _attn_tc_case(cfg["nh"], cfg["nkv"], cfg["hd"], cfg["window"], befores, [1] * 5, seed=cfg["hd"] + 7,
                        slices=slices, kernel="mma")
    assert err <= 2 ** -7, (cfg, slices, err)


@pytest.mark.parametrize("cfg", [dict(nh=8, nkv=2, hd=128, window=0), dict(nh=8, nkv=1, hd=64, window=0),
                                 dict(nh=2, nkv=2, hd=256, window=0), dict(nh=6, nkv=2, hd=64, window=50),
                                 dict(nh=32, nkv=2, hd=128, window=0)])
@pytest.mark.parametrize("slices", [None, 1, 3])
def test_attn_decode_tma(cfg, slices):
    """The decode kernel fed by TMA into swizzled shared memory, against the same oracle."""
    befores = [0, 63, 64, 300, 700]
    err = _attn_tc_case(cfg["nh"], cfg["nkv"], cfg["hd"], cfg["window"], befores, [1] * 5, seed=cfg["hd"] + 11,
                        slices=slices, kernel="tma")
    assert err <= 2 ** -7, (cfg, slices, err)


@pytest.mark.parametrize("hd", [64, 128])
@pytest.mark.parametrize("kernel", ["mma", "tma", "tc"])
@pytest.mark.parametrize("slices", [None, 1, 2])
def test_decode_attention_on_a_wrapped_window_ring(kernel, hd, slices):
    """A window of 100 kept in a ring of two pages (128 positions): position p lies at p mod 128, so once a
    sequence is past 128 the page that takes the new position also holds the window's oldest keys, and the
    first and the last key tile of a step are one physical page.  Only the window's mask and the zeroing of
    values past the sequence's end keep old from new."""
    for befores in ([127, 130, 200, 257], [128, 191, 192, 319], [63, 64, 100, 511]):
        err = _attn_tc_case(8, 2, hd, 100, befores, [1] * 4, seed=hd + 31, slices=slices, ring_pages=2, kernel=kernel)
        assert err <= 2 ** -7, (kernel, hd, slices, befores, err)


@pytest.mark.parametrize("hd", [48, 64, 128])
def test_decode_attention_mma_on_a_ring_of_one_page(hd):
    for befores in ([40, 63, 64, 65], [127, 128, 200, 1000]):
        err = _attn_tc_case(6, 3, hd, 33, befores, [1] * 4, seed=hd + 33, ring_pages=1, kernel="mma")
        assert err <= 2 ** -7, (hd, befores, err)
        if hd % 64 == 0:
            err = _attn_tc_case(6, 3, hd, 33, befores, [1] * 4, seed=hd + 34, ring_pages=1, kernel="tma", slices=2)
            assert err <= 2 ** -7, (hd, befores, err)


@pytest.mark.parametrize("kernel,wide", [("mma", 0), (None, 0), (None, 2)])
@pytest.mark.parametrize("hd", [64, 128])
def test_prompt_attention_on_a_wrapped_window_ring(kernel, wide, hd):
    """Continued prompts whose new tokens wrap around a ring of two pages: window 100, up to 29 new tokens
    (window + new tokens - 1 = 128 positions must be held), for the mma.sync and both tcgen05 kernels."""
    from ultima_b200.kernels import attn_tc
    was = attn_tc.WIDE
    attn_tc.set_wide(wide)
    try:
        for befores, news in (([127, 200, 257, 60], [20, 29, 5, 29]), ([100, 120, 128, 500], [29, 8, 29, 1])):
            err = _attn_tc_case(4, 2, hd, 100, befores, news, seed=hd + 35, ring_pages=2, kernel=kernel)
            assert err <= 2 ** -7, (kernel, wide, hd, befores, news, err)
    finally:
        attn_tc.set_wide(was)


@pytest.mark.parametrize("cfg", [dict(nh=8, nkv=2, hd=128, window=0, norm=True, rot=True),
                                 dict(nh=8, nkv=1, hd=64, window=0, norm=True, rot=True),
                                 dict(nh=2, nkv=2, hd=256, window=0, norm=False, rot=True),
                                 dict(nh=6, nkv=2, hd=64, window=50, norm=True, rot=False),
                                 dict(nh=32, nkv=2, hd=128, window=0, norm=True, rot=True)])
@pytest.mark.parametrize("slices", [None, 1, 3])
@pytest.mark.parametrize("owner", [True, False])
@pytest.mark.parametrize("wrapped", [False, True])
def test_attn_decode_from_the_projection_slices(cfg, slices, owner, wrapped):
    """The decode kernel that sums the slices of the fused projection, prepares q and the new key and
    writes the cache itself gives, bit for bit, what qk_prepare followed by the decode kernel gives:
    the output and the cache.  Without ownership of the cache it writes nothing and reads what is there.
    ``wrapped``: a window of 100 in a ring of two pages, sequences past the ring's end, so that the page
    of the new position is also the page of the window's oldest keys."""
    from ultima_b200.kernels import attn_tc
    from ultima_b200.engine import Runtime
    ops = _ops()
    rt = Runtime(DEV, torch.bfloat16)
    nh, nkv, hd, window = cfg["nh"], cfg["nkv"], cfg["hd"], cfg["window"]
    befores = [0, 63, 64, 300, 700]
    ring_pages = 12
    if wrapped:
        window, ring_pages, befores = 100, 2, [127, 130, 200, 257, 64]
    n = len(befores)
    lens = [b + 1 for b in befores]
    kc, vc, table, _ = _paged(n, lens, nkv, hd, torch.bfloat16, ring_pages, seed=hd + 21)
    g = torch.Generator().manual_seed(hd + 22)
    P, W = 3, (nh + 2 * nkv) * hd
    parts = (torch.randn(P, n, W, generator=g) * 0.6).to(DEV)
    qw = (1 + 0.1 * torch.randn(hd, generator=g)).to(DEV) if cfg["norm"] else None
    kw = (1 + 0.1 * torch.randn(hd, generator=g)).to(DEV) if cfg["norm"] else None
    cos = sin = None
    if cfg["rot"]:
        ang = torch.rand(800, hd // 2, generator=g) * 6.28
        cos, sin = torch.cos(ang).to(DEV), torch.sin(ang).to(DEV)
    b = _B()
    b.seq_start = torch.arange(n + 1, dtype=torch.int32, device=DEV)
    b.seq_before = torch.tensor(befores, dtype=torch.int32, device=DEV)
    b.n_seqs, b.max_new, b.max_after = n, 1, max(lens)
    tok_pos = b.seq_before.clone()
    tok_seq = torch.arange(n, dtype=torch.int32, device=DEV)
    eps = 1e-5
    # the two kernels
    kv_a = _KV(kc.clone(), vc.clone(), table, ring_pages * 64, window or None)
    kv_a.owner = owner
    q = torch.empty(n, nh * hd, dtype=torch.bfloat16, device=DEV)
    ops.qk_prepare(parts, qw, kw, cos, sin, tok_pos, tok_seq, kv_a.k, kv_a.v, table, kv_a.ring, 64, nh, nkv, hd, eps,
                   write_kv=owner, q_out=q)
    out_a = torch.full((n, nh * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
    attn_tc.attention(q, kv_a, out_a, b, nh, nkv, hd, 1 / math.sqrt(hd), rt, slices=slices, kernel="tma")
    # the one kernel
    kv_b = _KV(kc.clone(), vc.clone(), table, ring_pages * 64, window or None)
    kv_b.owner = owner
    out_b = torch.full((n, nh * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
    assert attn_tc.decode_from_qkv(parts, qw, kw, cos, sin, eps, kv_b, out_b, b, nh, nkv, hd, 1 / math.sqrt(hd), rt,
                                   slices=slices, force=True)
    torch.cuda.synchronize()
    rt.check_status()
    assert torch.isfinite(out_b).all()
    assert torch.equal(out_a, out_b), (cfg, slices, owner, (out_a.float() - out_b.float()).abs().max().item())
    same = lambda x, y: torch.equal(x.view(torch.int16), y.view(torch.int16))       # NaN-filled spare rows too
    assert same(kv_a.k, kv_b.k) and same(kv_a.v, kv_b.v)
    if not owner:
        assert same(kv_b.k, kc) and same(kv_b.v, vc)
    else:
        assert not same(kv_b.k, kc)


def test_gemm_tc_partial_products_and_their_consumers():
    """K cut into slices written side by side; qk_prepare and silu_mul add the slices up."""
    gemm_tc, rt = _tc()
    ops = _ops()
    g = torch.Generator().manual_seed(4)
    T, K, nh, nkv, hd = 5, 1024, 4, 2, 128
    N = (nh + 2 * nkv) * hd
    a = torch.randn(T, K, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    parts = torch.full((4, T, N), float("nan"), device=DEV)
    gemm_tc.gemm(a, w, parts, ops.EPI_STORE, None, rt, splits=4)
    ref = a.double() @ w.double().T
    assert rel_err(parts.sum(0), ref) <= 1e-4
    assert gemm_tc.store_splits(8, 6144, 4096) > 1 and gemm_tc.store_splits(2048, 6144, 4096) == 1
    # qk_prepare over the slices == qk_prepare over their sum
    table = torch.tensor([[0], [1]], dtype=torch.int32, device=DEV)
    pos = torch.tensor([0, 1, 2, 0, 1], dtype=torch.int32, device=DEV)
    seq = torch.tensor([0, 0, 0, 1, 1], dtype=torch.int32, device=DEV)
    qw = (1 + 0.1 * torch.randn(hd, generator=g)).to(DEV)
    kw = (1 + 0.1 * torch.randn(hd, generator=g)).to(DEV)
    cos = torch.cos(torch.arange(8)[:, None] * torch.arange(hd // 2)[None] * 0.1).float().to(DEV)
    sin = torch.sin(torch.arange(8)[:, None] * torch.arange(hd // 2)[None] * 0.1).float().to(DEV)
    # the same rows through the kernel for any head size (48) give the same numbers where they overlap:
    # covered by test_qk_prepare_norm_rotation_and_cache_write; here the slices are what is checked
    outs = []
    for src in (parts, parts.sum(0).contiguous()):
        kc = torch.zeros(2, nkv, 64, hd, dtype=torch.bfloat16, device=DEV)
        vc = torch.zeros_like(kc)
        q = torch.zeros(T, nh * hd, dtype=torch.bfloat16, device=DEV)
        ops.qk_prepare(src, qw, kw, cos, sin, pos, seq, kc, vc, table, 64, 64, nh, nkv, hd, 1e-6, q_out=q)
        outs.append((q, kc, vc))
    for x, y in zip(outs[0], outs[1]):
        assert rel_err(x, y.double()) <= 2 ** -7
    assert float(outs[0][0].abs().sum()) > 0 and float(outs[0][1].abs().sum()) > 0
    # silu_mul over slices
    F = 96
    gu = torch.randn(3, T, 2 * F, generator=g).to(DEV)
    out = torch.empty(T, F, dtype=torch.bfloat16, device=DEV)
    ops.silu_mul(gu, out)
    sd = gu.double().sum(0)
    assert rel_err(out, sd[:, :F] / (1 + torch.exp(-sd[:, :F])) * sd[:, F:]) <= 2 ** -8


@pytest.mark.parametrize("shape", [(1, 64, 64), (9, 96, 320), (64, 4096, 256), (130, 512, 192), (300, 1024, 640)])
def test_gemm_tc_interleaved_gate_product(shape):
    """Blocks of 64 gate rows and 64 up rows alternate in one matrix."""
    gemm_tc, rt = _tc()
    ops = _ops()
    T, K, F = shape
    g = torch.Generator().manual_seed(F + T)
    a = torch.randn(T, K, generator=g).to(torch.bfloat16).to(DEV)
    wg = (torch.randn(F, K, generator=g) * 0.05).to(torch.bfloat16)
    wu = (torch.randn(F, K, generator=g) * 0.05).to(torch.bfloat16)
    il = torch.stack([wg.view(F // 64, 64, K), wu.view(F // 64, 64, K)], dim=1).reshape(2 * F, K).contiguous().to(DEV)
    out = torch.full((T, F), float("nan"), dtype=torch.bfloat16, device=DEV)
    assert gemm_tc.accepts(a, il, out, ops.EPI_SWIGLU_IL, None)
    gemm_tc.gemm(a, il, out, ops.EPI_SWIGLU_IL, None, rt)
    torch.cuda.synchronize()
    gemm_tc.check_error(rt)
    gt, up = a.double().cpu() @ wg.double().T, a.double().cpu() @ wu.double().T
    assert rel_err(out, gt / (1 + torch.exp(-gt)) * up) <= 2 ** -8, shape


@pytest.mark.parametrize("pairs", [False, True])
@pytest.mark.parametrize("case", [("store", 2500, 1024, 1200), ("add", 2500, 512, 2100), ("add", 5000, 128, 1100), ("gate_il", 1700, 256, 1280),
                                  ("gate_two", 1100, 320, 1300), ("store_f32", 700, 128, 5000),
                                  ("store", 2600, 192, 2100), ("gate_il", 2100, 128, 2560), ("store_f32", 1300, 64, 3300),
                                  ("add", 2049, 4096, 4096)])
def test_gemm_tc_many_tiles_a_cta(case, pairs, monkeypatch):
    """More tiles than SMs: CTAs stay and walk over tiles with two accumulators in turn; with
    ``pairs`` two CTAs share a tile of 256 weight rows by 256 tokens where there are enough tiles
    (the last six cases but one), else the same kernel as without."""
    gemm_tc, rt = _tc()
    ops = _ops()
    kind, T, K, N = case
    monkeypatch.setattr(gemm_tc, "USE_PAIRS", pairs)
    if pairs and case[1:] in ((2600, 192, 2100), (2100, 128, 2560), (1300, 64, 3300), (2049, 4096, 4096), (5000, 128, 1100)):
        assert gemm_tc.pairs(T, N, 1, ops.EPI_STORE)
    g = torch.Generator().manual_seed(T)
    a = torch.randn(T, K, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    ref = a.double() @ w.double().T
    tol = max(2e-6, K * 2.0 ** -25)
    if kind == "store":
        out = torch.full((T, N), float("nan"), dtype=torch.bfloat16, device=DEV)
        gemm_tc.gemm(a, w, out, ops.EPI_STORE, None, rt)
        assert rel_err(out, ref) <= 2 ** -8
    elif kind == "store_f32":
        out = torch.full((T, N), float("nan"), dtype=torch.float32, device=DEV)
        gemm_tc.gemm(a, w, out, ops.EPI_STORE, None, rt)
        assert rel_err(out, ref) <= tol
    elif kind == "add":
        acc = torch.randn(T, N, generator=g).to(DEV)
        want = acc.double() + ref
        gemm_tc.gemm(a, w, acc, ops.EPI_ADD, None, rt)
        assert rel_err(acc, want) <= tol
    elif kind == "gate_il":
        F = N // 2
        il = torch.stack([w[:F].view(F // 64, 64, K), w[F:].view(F // 64, 64, K)], dim=1).reshape(N, K).contiguous()
        out = torch.full((T, F), float("nan"), dtype=torch.bfloat16, device=DEV)
        gemm_tc.gemm(a, il, out, ops.EPI_SWIGLU_IL, None, rt)
        assert rel_err(out, ref[:, :F] / (1 + torch.exp(-ref[:, :F])) * ref[:, F:]) <= 2 ** -8
    else:
        F = N // 2
        out = torch.full((T, F), float("nan"), dtype=torch.bfloat16, device=DEV)
        gemm_tc.gemm(a, w[:F], out, ops.EPI_SWIGLU, w[F:], rt)
        assert rel_err(out, ref[:, :F] / (1 + torch.exp(-ref[:, :F])) * ref[:, F:]) <= 2 ** -8
    torch.cuda.synchronize()
    gemm_tc.check_error(rt)


@pytest.mark.parametrize("kernel,new", [("mma", 1), ("mma", 2), ("tma", 1), (None, 2), ("tc", 1)])
def test_tensor_core_attention_finds_a_far_key_and_respects_the_window_edge(kernel, new):
    """As for the plain kernel: one key among hundreds stands out; a window that ends one short of it
    must not see it, a window that just reaches it must.  ``new`` = 1 runs the decode kernels, 2 the
    prompt kernels (mma.sync, TMA-fed, tcgen05)."""
    from ultima_b200.kernels import attn_tc
    from ultima_b200.engine import Runtime
    rt = Runtime(DEV, torch.bfloat16)
    nh, nkv, hd, n = 2, 1, 64, 700
    g = torch.Generator().manual_seed(3)
    k = torch.randn(n, nkv, hd, generator=g) * 0.1
    v = torch.randn(n, nkv, hd, generator=g) * 0.1
    qv = torch.randn(nh * hd, generator=g) * 0.1
    far = 213
    k[far, 0] = qv[:hd] * 400.0
    v[far, 0] = 5.0
    ring_pages = 11
    kc = torch.full((ring_pages, nkv, 64, hd), float("nan"), dtype=torch.bfloat16)
    vc = torch.full((ring_pages, nkv, 64, hd), float("nan"), dtype=torch.bfloat16)
    for p_ in range(n):
        kc[p_ // 64, :, p_ % 64], vc[p_ // 64, :, p_ % 64] = k[p_].to(torch.bfloat16), v[p_].to(torch.bfloat16)
    table = torch.arange(ring_pages, dtype=torch.int32).view(1, -1).to(DEV)
    q = qv[None].repeat(new, 1).to(torch.bfloat16).to(DEV)
    b = _B()
    b.seq_start = torch.tensor([0, new], dtype=torch.int32, device=DEV)
    b.seq_before = torch.tensor([n - new], dtype=torch.int32, device=DEV)
    b.n_seqs, b.max_new, b.max_after = 1, new, n

    def run(window):
        out = torch.full((new, nh * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
        kv = _KV(kc.to(DEV), vc.to(DEV), table, ring_pages * 64, window or None)
        attn_tc.attention(q, kv, out, b, nh, nkv, hd, 1 / math.sqrt(hd), rt, kernel=kernel)
        torch.cuda.synchronize()
        rt.check_status()
        return out[new - 1, :hd].float()                       # head 0 of the token at position n - 1

    assert float(run(0).min()) > 4.9
    assert float(run(n - 1 - far).abs().max()) < 1.0           # the window ends one short of the far key
    assert float(run(n - far).min()) > 4.9                     # the window just reaches it
