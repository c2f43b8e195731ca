// Device code shared by the attention kernels on mma.sync (attn_mma.cu) and by the decode kernel
// that runs a whole stack of layers (decode_stack.cu), for one head size fixed at compile time
// (-DHEAD_DIM=...): the tile arithmetic of flash attention (scores, running softmax, weighted
// values) over tiles in padded or in 128-byte-swizzled shared memory, and the preparation of
// queries and the new key from the fused projection's float32 result.
#pragma once
#include "common.cuh"

#ifndef HEAD_DIM
#define HEAD_DIM 128
#endif
static_assert(HEAD_DIM % 16 == 0 && HEAD_DIM >= 16 && HEAD_DIM <= 256, "head size: a multiple of 16 up to 256");

constexpr int HD = HEAD_DIM;
constexpr int LDS = HD + 8;                 // shared-memory row stride (elements): no bank conflicts for ldmatrix
constexpr int KT = 64;                      // keys a tile = positions a page
constexpr int NTHREADS = 128;
#ifndef ATTN_DSTAGES
#define ATTN_DSTAGES 2
#endif
#ifndef ATTN_ALIAS
#define ATTN_ALIAS 0        // 1: the merge buffer lies over the K/V ring (less shared memory, a third CTA an SM: measured slower)
#endif
constexpr int DSTAGES = ATTN_DSTAGES;       // K/V tiles in the decode kernel's ring
constexpr int KSTEPS = HD / 16;
constexpr int DTILES = HD / 8;

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x2(uint32_t addr, uint32_t& r0, uint32_t& r1) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0, %1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float* d, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Load one page (64 positions of one KV head) of K and V into shared memory; positions above
// ``last_pos`` become zeros.  ``base`` is the absolute position of the tile's first key.
__device__ __forceinline__ void load_kv_tile(bf16* Ks, bf16* Vs, const bf16* __restrict__ kc, const bf16* __restrict__ vc,
                                             const PagedKV& c, int seq, int kvh, int base, int last_pos, int tid) {
    const long long off = paged_offset(c, seq, base, kvh);            // first position of the page
    constexpr int CH = HD / 8;                                         // 16-byte pieces a row
    for (int i = tid; i < KT * CH; i += NTHREADS) {
        const int r = i / CH, ch = i % CH;
        bf16* kd = Ks + r * LDS + ch * 8;
        bf16* vd = Vs + r * LDS + ch * 8;
        if (base + r <= last_pos) {
            cp_async16(kd, kc + off + (long long)r * HD + ch * 8);
            cp_async16(vd, vc + off + (long long)r * HD + ch * 8);
        } else {
            *reinterpret_cast<uint4*>(kd) = make_uint4(0, 0, 0, 0);
            *reinterpret_cast<uint4*>(vd) = make_uint4(0, 0, 0, 0);
        }
    }
}

// Scores of 16 rows against ``NT`` groups of 8 keys starting at key row ``key0`` of the K tile.
template <int NT>
__device__ __forceinline__ void scores(float (*s)[4], const bf16* Qs, int q_row0, const bf16* Ks, int key0, int lane) {
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) { s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f; }
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) {
        uint32_t a[4];
        ldsm_x4(smem_addr(Qs + (q_row0 + (lane & 15)) * LDS + ks * 16 + (lane >> 4) * 8), a[0], a[1], a[2], a[3]);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            uint32_t b0, b1;
            ldsm_x2(smem_addr(Ks + (key0 + nt * 8 + (lane & 7)) * LDS + ks * 16 + ((lane >> 3) & 1) * 8), b0, b1);
            mma_bf16(s[nt], a, b0, b1);
        }
    }
}

// o += P V for 16 rows, P being the probabilities of ``NT`` groups of 8 keys (NT even) held in
// the accumulator layout of ``scores``; the V rows start at ``key0`` of the V tile.
template <int NT>
__device__ __forceinline__ void weighted_values(float (*o)[4], const float (*s)[4], const bf16* Vs, int key0, int lane) {
#pragma unroll
    for (int kk = 0; kk < NT / 2; ++kk) {
        uint32_t a[4];
        a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
        a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
        a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
        a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
        for (int dt = 0; dt < DTILES; dt += 2) {
            uint32_t b0, b1, b2, b3;
            const int row = key0 + kk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
            const int col = dt * 8 + (lane >> 4) * 8;
            ldsm_x4_trans(smem_addr(Vs + row * LDS + col), b0, b1, b2, b3);
            mma_bf16(o[dt], a, b0, b1);
            mma_bf16(o[dt + 1], a, b2, b3);
        }
    }
}

// One step of the running softmax over the masked scores of NT key groups; scores come in raw
// (q.k) and leave as probabilities relative to the new maximum.  c = scale * log2(e).
template <int NT>
__device__ __forceinline__ void softmax_step(float (*s)[4], float (*o)[4], float* m, float* l, float c,
                                             const int* row_pos, bool const* row_ok, int key_pos0, int window, int lane) {
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int r = e >> 1;
            const int kp = key_pos0 + nt * 8 + (lane & 3) * 2 + (e & 1);
            const bool ok = row_ok[r] && kp <= row_pos[r] && (window <= 0 || kp > row_pos[r] - window);
            const float v = ok ? s[nt][e] * c : -INFINITY;
            s[nt][e] = v;
            mx[r] = fmaxf(mx[r], v);
        }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
    }
    float corr[2], base[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const float m_new = fmaxf(m[r], mx[r]);
        base[r] = m_new == -INFINITY ? 0.f : m_new;           // a row with nothing visible yet
        corr[r] = exp2f(m[r] - base[r]);                      // 0 when m is -inf
        m[r] = m_new;
    }
    float sum[2] = {0.f, 0.f};
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float p = exp2f(s[nt][e] - base[e >> 1]);
            s[nt][e] = p;
            sum[e >> 1] += p;
        }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], 1);
        sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], 2);
        l[r] = l[r] * corr[r] + sum[r];
    }
#pragma unroll
    for (int dt = 0; dt < DTILES; ++dt) {
        o[dt][0] *= corr[0]; o[dt][1] *= corr[0];
        o[dt][2] *= corr[1]; o[dt][3] *= corr[1];
    }
}


#if HEAD_DIM % 64 == 0
#include "tc_common.cuh"

#ifndef ATTN_TSTAGES
#define ATTN_TSTAGES 3
#endif
constexpr int TSTAGES = ATTN_TSTAGES;
constexpr int NBLK = HD / 64;                       // 64-column blocks of a row
constexpr int PAGE_BYTES = KT * HD * 2;             // one K or V page of one KV head
constexpr int BLK_BYTES = KT * 128;                 // one 64-column block of a page
constexpr int TMA_THREADS = 160;

// byte offset of element (row, col) in a tile stored as NBLK swizzled blocks of [64 rows][128 bytes]
__device__ __forceinline__ uint32_t swz(int row, int col) {
    return (uint32_t)((col >> 6) * BLK_BYTES + row * 128 + ((((col & 63) >> 3) ^ (row & 7)) << 4) + ((col & 7) << 1));
}

template <int NT>
__device__ __forceinline__ void scores_swz(float (*s)[4], const bf16* Qs, uint32_t k_base, int key0, int lane) {
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) { s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f; }
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) {
        uint32_t a[4];
        ldsm_x4(smem_addr(Qs + (lane & 15) * LDS + ks * 16 + (lane >> 4) * 8), a[0], a[1], a[2], a[3]);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            uint32_t b0, b1;
            ldsm_x2(k_base + swz(key0 + nt * 8 + (lane & 7), ks * 16 + ((lane >> 3) & 1) * 8), b0, b1);
            mma_bf16(s[nt], a, b0, b1);
        }
    }
}
template <int NT>
__device__ __forceinline__ void weighted_values_swz(float (*o)[4], const float (*s)[4], uint32_t v_base, int key0, int lane) {
#pragma unroll
    for (int kk = 0; kk < NT / 2; ++kk) {
        uint32_t a[4];
        a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
        a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
        a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
        a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
        for (int dt = 0; dt < DTILES; dt += 2) {
            uint32_t b0, b1, b2, b3;
            const int row = key0 + kk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
            const int col = dt * 8 + (lane >> 4) * 8;
            ldsm_x4_trans(v_base + swz(row, col), b0, b1, b2, b3);
            mma_bf16(o[dt], a, b0, b1);
            mma_bf16(o[dt + 1], a, b2, b3);
        }
    }
}

// With ``qkv`` set the kernel also does what qk_prepare does for a step of one token a sequence: a
// CTA sums the partial results of the fused projection for its own query heads, norms and rotates
// them straight into shared memory, and the CTA that reads the page of the new position does the
// same for the new key (and copies the new value), writes both into the cache for later steps and
// puts them into its own copy of the page.  q never goes through global memory, and the kernel
// between the projection and the attention is gone.
struct FusedQKV {
    const float* qkv;            // [n_parts][tokens, (nh + 2 nkv) * HD] float32; null: q is read from a.q
    int n_parts; long long part_stride;
    const float* qw; const float* kw;        // [HD] norm weights or null
    const float* cs; const float* sn;        // [max_pos, HD / 2] or null
    float eps;
    bf16* kcache; bf16* vcache;              // where the new key and value go; null: the cache is another layer's
};

constexpr bool FUSABLE = HD == 64 || HD == 128 || HD == 256;
constexpr int FE = FUSABLE ? HD / 32 : 2;       // elements of a head a lane holds, neighbours; the lower 16
                                                // lanes the first half of the head, the upper 16 the second

// The sums of the partial results of NSRC heads of the fused projection's row, a lane's FE elements
// of each: four parts of every head are in flight before the first add, and they are added in
// their order.
template <int NSRC>
__device__ __forceinline__ void fused_sums(const FusedQKV& f, const float* const* src, int lane, float (*v)[FE]) {
    for (int p0 = 0; p0 < f.n_parts; p0 += 4) {
        float part[NSRC][4][FE];
#pragma unroll
        for (int s = 0; s < NSRC; ++s) {
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                if (p0 + u < f.n_parts) load_vec<float, FE>(src[s] + (long long)(p0 + u) * f.part_stride + lane * FE, part[s][u]);
                else {
#pragma unroll
                    for (int i = 0; i < FE; ++i) part[s][u][i] = 0.f;
                }
            }
        }
#pragma unroll
        for (int s = 0; s < NSRC; ++s) {
#pragma unroll
            for (int u = 0; u < 4; ++u) {
#pragma unroll
                for (int i = 0; i < FE; ++i) v[s][i] = (p0 == 0 && u == 0) ? part[s][u][i] : v[s][i] + part[s][u][i];
            }
        }
    }
}

// Norm with ``w`` (or not) and rotation by (co, si) (or not) of one head held FE elements a lane.
__device__ __forceinline__ void fused_finish(const FusedQKV& f, const float* w, bool rotate, const float* co,
                                             const float* si, int lane, float* v) {
    if (w) {
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < FE; ++i) ss += v[i] * v[i];
        ss = warp_sum(ss);
        const float inv = inv_rms(ss, (float)HD, f.eps);
#pragma unroll
        for (int i = 0; i < FE; ++i) v[i] = v[i] * w[i] * inv;
    }
    if (rotate) {
        const bool upper = lane >= 16;
#pragma unroll
        for (int i = 0; i < FE; ++i) {
            const float other = __shfl_xor_sync(0xffffffffu, v[i], 16);
            v[i] = upper ? other * si[i] + v[i] * co[i] : v[i] * co[i] - other * si[i];
        }
    }
}

#endif   // HEAD_DIM % 64 == 0
