"""The tests' own copy of the package's random-weight generator: element ``i`` of a tensor is a
function of (key, i), with the key made from the seed and the tensor's name.

It shares no code with the package.  Where the package's numpy version works on whole arrays,
this one is written value by value with numpy's float32 scalars, each line one correctly rounded
operation; ``normal_array`` is the same thing over arrays for tensors of real size.  The three
(this, weights/random_init.py and the CUDA kernel) must agree bit for bit, which
tests/test_random_weights.py and tests/test_kernels_gpu.py check.
"""
import hashlib

import numpy as np

F = np.float32
MASK = (1 << 64) - 1


def fb(bits: int) -> np.float32:
    return np.array([bits], dtype=np.uint32).view(np.float32)[0]


LN2, SQRT2, HALF_PI = fb(0x3F317218), fb(0x3FB504F3), fb(0x3FC90FDB)
LOG_ODD = [fb(0x3DBA2E8C), fb(0x3DE38E39), fb(0x3E124925), fb(0x3E4CCCCD), fb(0x3EAAAAAB)]     # 1/11 ... 1/3
SIN_FACT = [fb(0x3638EF1D), fb(0x39500D01), fb(0x3C088889), fb(0x3E2AAAAB)]                    # 1/9! ... 1/3!
COS_FACT = [fb(0x3493F27E), fb(0x37D00D01), fb(0x3AB60B61), fb(0x3D2AAAAB)]                    # 1/10! ... 1/4!


def tensor_key(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode("utf-8")).digest()
    return int.from_bytes(h[:8], "little") & ((1 << 63) - 1)


def mix64(z: int) -> int:
    z = (z + 0x9E3779B97F4A7C15) & MASK
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & MASK
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & MASK
    return z ^ (z >> 31)


def normal_one(key: int, i: int) -> np.float32:
    """One standard normal draw, scalar arithmetic."""
    r = mix64(key ^ mix64(i))
    u1 = F(F(F(r >> 41) + F(0.5)) * fb(0x34000000))
    bits = int(np.array([u1], dtype=np.float32).view(np.uint32)[0])
    e = (bits >> 23) - 127
    m = fb((bits & 0x7FFFFF) | 0x3F800000)
    if m > SQRT2:
        m = F(m * F(0.5))
        e += 1
    s = F(F(m - F(1.0)) / F(m + F(1.0)))
    s2 = F(s * s)
    p = LOG_ODD[0]
    for c in LOG_ODD[1:]:
        p = F(F(p * s2) + c)
    p = F(F(p * s2) + F(1.0))
    ln_m = F(F(F(2.0) * s) * p)
    ln_u = F(F(F(e) * LN2) + ln_m)
    rad = np.sqrt(F(F(-2.0) * ln_u))
    t = (r >> 16) & 0xFFFFFF
    quad, rest = t >> 22, t & 0x3FFFFF
    fold = rest > 0x200000
    fr = 0x400000 - rest if fold else rest
    x = F(F(F(fr) * fb(0x34800000)) * HALF_PI)
    x2 = F(x * x)
    sn = SIN_FACT[0]
    for c in SIN_FACT[1:]:
        sn = F(c - F(sn * x2))
    sn = F(F(F(1.0) - F(sn * x2)) * x)
    cs = COS_FACT[0]
    for c in COS_FACT[1:]:
        cs = F(c - F(cs * x2))
    cs = F(F(0.5) - F(cs * x2))
    cs = F(F(1.0) - F(cs * x2))
    sin_q, cos_q = (cs, sn) if fold else (sn, cs)
    c = (cos_q, -sin_q, -cos_q, sin_q)[quad]
    return F(rad * c)


def normal_array(key: int, n: int, chunk: int = 1 << 16) -> np.ndarray:
    """The same draws for elements 0 .. n - 1, over arrays."""
    out = np.empty(n, dtype=np.float32)
    u64, u32 = np.uint64, np.uint32
    for a in range(0, n, chunk):
        b = min(n, a + chunk)
        with np.errstate(over="ignore"):
            def mix(z):
                z = z + u64(0x9E3779B97F4A7C15)
                z = (z ^ (z >> u64(30))) * u64(0xBF58476D1CE4E5B9)
                z = (z ^ (z >> u64(27))) * u64(0x94D049BB133111EB)
                return z ^ (z >> u64(31))
            r = mix(u64(key) ^ mix(np.arange(a, b, dtype=np.uint64)))
        u1 = ((r >> u64(41)).astype(F) + F(0.5)) * fb(0x34000000)
        bits = u1.view(u32)
        e = (bits >> u32(23)).astype(np.int32) - 127
        m = ((bits & u32(0x7FFFFF)) | u32(0x3F800000)).view(F)
        big = m > SQRT2
        m = np.where(big, m * F(0.5), m)
        e = np.where(big, e + 1, e).astype(np.int32)
        s = (m - F(1.0)) / (m + F(1.0))
        s2 = s * s
        p = np.full(b - a, LOG_ODD[0], dtype=F)
        for c in LOG_ODD[1:]:
            p = p * s2 + c
        p = p * s2 + F(1.0)
        ln_u = e.astype(F) * LN2 + (F(2.0) * s) * p
        rad = np.sqrt(F(-2.0) * ln_u)
        t = ((r >> u64(16)) & u64(0xFFFFFF)).astype(u32)
        quad, rest = t >> u32(22), t & u32(0x3FFFFF)
        fold = rest > u32(0x200000)
        fr = np.where(fold, u32(0x400000) - rest, rest)
        x = (fr.astype(F) * fb(0x34800000)) * HALF_PI
        x2 = x * x
        sn = np.full(b - a, SIN_FACT[0], dtype=F)
        for c in SIN_FACT[1:]:
            sn = c - sn * x2
        sn = (F(1.0) - sn * x2) * x
        cs = np.full(b - a, COS_FACT[0], dtype=F)
        for c in COS_FACT[1:]:
            cs = c - cs * x2
        cs = F(0.5) - cs * x2
        cs = F(1.0) - cs * x2
        sin_q, cos_q = np.where(fold, cs, sn), np.where(fold, sn, cs)
        out[a:b] = rad * np.select([quad == 0, quad == 1, quad == 2], [cos_q, -sin_q, -cos_q], sin_q)
    return out


def to_bfloat16_bits(x: np.ndarray) -> np.ndarray:
    """float32 -> the upper 16 bits after rounding to nearest even (no NaN among random weights)."""
    u = x.astype(np.float32).view(np.uint32)
    return ((u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) >> np.uint32(16)).astype(np.uint16)


def tensor(seed: int, name: str, shape, init, dtype: str = "float32") -> np.ndarray:
    """The package's random tensor ``name`` for ``seed``: float32 values, rounded to bfloat16 and
    widened again when ``dtype`` is "bfloat16" (what a bfloat16 model folder holds)."""
    n = int(np.prod(shape))
    z = normal_array(tensor_key(seed, name), n)
    shift = F(1.0) if init[0] == "one_plus_normal" else F(0.0)
    v = (shift + F(init[1]) * z).astype(np.float32)
    if dtype == "bfloat16":
        v = (to_bfloat16_bits(v).astype(np.uint32) << np.uint32(16)).view(np.float32)
    return v.reshape(shape)
