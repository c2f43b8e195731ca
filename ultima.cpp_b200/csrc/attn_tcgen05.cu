// Attention over the paged bfloat16 cache on the fifth-generation tensor cores, for prompts and for
// decode steps, for one head size fixed at compile time (-DHEAD_DIM=64 or 128).
//
// One CTA takes 128 rows of one KV head, a row being (token, query head of the group), and walks
// over the cache pages (64 keys) its rows may see.  Scores and the output live in tensor memory:
//   S_b = Q K^T     tcgen05.mma, both operands from shared memory (TMA, 128-byte swizzle), two
//                   score buffers so the next tile's scores are formed while this tile's are used
//   softmax         four warps, one thread a row: tcgen05.ld of the row's 64 scores, mask, running
//                   maximum and sum in float32, probabilities rounded to bfloat16 and stored back
//                   over the scores (tcgen05.st), two to a 32-bit column
//   O += P V        tcgen05.mma with P from tensor memory and V from shared memory (V is the
//                   N-major operand: rows of keys as TMA wrote them)
// The maximum a row's exponentials refer to is raised only when the true maximum has grown by more
// than 2^8 (then the row's output and sum are rescaled in tensor memory), so most tiles cost no
// pass over the output.  Rows of V the sequence has not reached are zeroed in shared memory.
// Warp 0 issues TMA, warp 1 issues MMAs and owns the tensor-memory allocation, warps 2-5 are the
// softmax.  Every wait has a time limit and raises a flag.  The issuing thread never waits for its
// own MMAs: they run in the order of their issue, so the scores of tile j+1 are queued right behind
// the product that reads the buffer they fall into.  Long prompts take a second kernel further
// down, attn_tc_wide_kernel, with 256 rows (two such tiles of rows) a CTA.
//
// The arithmetic restated is the reference's per-token loop (src/model/qwen_block.cpp:94-135):
// scores q.k * scale over the visible positions (p - window, p], max-shifted softmax, weighted
// sum of values, query head h on KV head h / (heads / kv heads).
#include "common.cuh"
#include "tc_common.cuh"

#ifndef HEAD_DIM
#define HEAD_DIM 128
#endif
static_assert(HEAD_DIM == 64 || HEAD_DIM == 128, "this kernel is built for head sizes 64 and 128");

constexpr int HD = HEAD_DIM;
constexpr int NB = HD / 64;                 // 64-column blocks of a row (one 128-byte swizzle span each)
constexpr int BM = 128;                     // rows a CTA
constexpr int BN = 64;                      // keys a tile = positions a page
constexpr int Q_BYTES = NB * BM * 128;
constexpr int KV_BYTES = NB * BN * 128;     // one K or V tile
constexpr int smem_bytes(int stages) { return Q_BYTES + 2 * stages * KV_BYTES + 1024 + 256; }
constexpr int TMEM_COLS = 256;              // S0 [0,64) S1 [64,128) O [128, 128 + HD)
constexpr int O_COL = 128;
constexpr float RESCALE_STEP = 8.0f;        // log2 units the reference maximum may lag behind
constexpr int NTHREADS = 192;
#ifndef DECODE_STAGES
#define DECODE_STAGES 4                     // K/V tiles in flight in the decode kernel (one CTA an SM)
#endif

typedef __nv_bfloat16 bf16;

struct TcAttnParams {
    bf16* out; long long o_stride;
    const int* seq_start; const int* seq_before; const int* table;
    int pages_per_seq, ring, nkv, group, window;
    float c;                                  // scale * log2(e)
    int* error;
    // decode (one new token a sequence, keys in slices): unnormalised partial results
    float* part_o; float* part_ml; int n_slices, nh;
    int n_seqs, n_row_tiles;                  // prompts: the grid is n_row_tiles * n_seqs * nkv blocks
};

__host__ __device__ constexpr uint32_t idesc_bf16(int m, int n, int b_mn_major) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)b_mn_major << 16) | ((uint32_t)(n >> 3) << 17) |
           ((uint32_t)(m >> 4) << 24);
}
// 2^x by the special-function unit (relative error 2^-22; -inf gives 0)
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// Two float32 in a 64-bit register and the arithmetic on such pairs (one instruction for both), and the
// maximum of three.
__device__ __forceinline__ uint64_t pair_of(float a, float b) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
    return r;
}
__device__ __forceinline__ void halves_of(uint64_t v, float& a, float& b) { asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v)); }
__device__ __forceinline__ uint64_t fma_pair(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ uint64_t add_pair(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
// V tile as the N-major B operand: rows of 128 bytes are keys, 8 keys a swizzle atom (1024 bytes)
__device__ __forceinline__ uint64_t make_desc_mn(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
    d |= (uint64_t)((BN * 128) >> 4) << 16;                // next 64 columns
    d |= (uint64_t)(1024 >> 4) << 32;                      // next 8 keys
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

// KV_STAGES: K/V tiles in flight.  DECODE: one new token a sequence; blockIdx.x is then a slice of the
// key range instead of a tile of rows, and with several slices the CTA writes (reference maximum,
// sum, unnormalised output) for attn_tc_combine_kernel.
template <int KV_STAGES, bool DECODE>
__global__ void __launch_bounds__(NTHREADS)
attn_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
               const __grid_constant__ CUtensorMap map_v, TcAttnParams p) {
    extern __shared__ uint8_t smem_raw[];
    // prompts: a one-dimensional grid numbered so that the blocks with the most keys to visit (the
    // last tiles of the rows, of every sequence and KV head) are handed out first
    const int per_tile = p.n_seqs * p.nkv;
    const int seq = DECODE ? blockIdx.y : (blockIdx.x % per_tile) / p.nkv;
    const int kvh = DECODE ? blockIdx.z : blockIdx.x % p.nkv;
    const int q0 = p.seq_start[seq], q_len = p.seq_start[seq + 1] - q0, before = p.seq_before[seq];
    const int G = p.group;
    const int TPB = BM / G;                                // tokens a tile: TPB * G of the 128 rows are in use
    const int tile = DECODE ? 0 : p.n_row_tiles - 1 - blockIdx.x / per_tile;
    const int tok_first = tile * TPB;
    if (tok_first >= q_len) return;                        // (a block that ends counts as one that has let its dependents go)

    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* q_s = smem;
    uint8_t* k_s = q_s + Q_BYTES;
    uint8_t* v_s = k_s + KV_STAGES * KV_BYTES;
    uint64_t* bars = (uint64_t*)(v_s + KV_STAGES * KV_BYTES);
    uint64_t* q_full = bars;
    uint64_t* k_full = bars + 1;
    uint64_t* k_empty = k_full + KV_STAGES;
    uint64_t* v_full = k_empty + KV_STAGES;
    uint64_t* v_empty = v_full + KV_STAGES;
    uint64_t* s_full = v_empty + KV_STAGES;               // [2]
    uint64_t* p_full = s_full + 2;                        // [2]
    uint64_t* pv_done = p_full + 2;                       // [2]
    uint32_t* tmem_slot = (uint32_t*)(pv_done + 2);
    volatile int* err = (volatile int*)(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int last_pos = before + q_len - 1;
    const int tok_last = min(q_len - 1, tok_first + TPB - 1);
    const int pos_hi = before + tok_last;
    int pos_lo = 0;
    if (p.window > 0) pos_lo = max(0, before + tok_first - p.window + 1);
    int t_lo = pos_lo / BN, n_tiles = pos_hi / BN - t_lo + 1;
    if (DECODE) {                                          // this CTA's slice of the tiles (may be empty)
        const int per = (n_tiles + p.n_slices - 1) / p.n_slices;
        const int first = min(n_tiles, (int)blockIdx.x * per);
        n_tiles = min(n_tiles - first, per);
        t_lo += first;
    }

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int s = 0; s < KV_STAGES; ++s) {
            mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1);
            mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) { mbar_init(&s_full[b], 1); mbar_init(&p_full[b], 4); mbar_init(&pv_done[b], 1); }
        *err = 0;
        fence_barrier_init();
    }
    if (warp == 1) { tmem_alloc(tmem_slot, TMEM_COLS); tmem_relinquish(); }
    if (warp == 0 && lane == 0) { prefetch_tmap(&map_q); prefetch_tmap(&map_k); prefetch_tmap(&map_v); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // Dependents are let go only now that this block holds its tensor memory: a dependent product
    // allocates its own before it waits for this grid's end and keeps it until then, so a block of
    // this grid that still had to allocate beside it could wait for columns that never come free.
    pdl_trigger();
    pdl_wait();

    if (warp == 0) {
        // ---------------- TMA ----------------
        if (lane == 0) {
            if (n_tiles > 0) {
                mbar_expect_tx(q_full, NB * TPB * G * 128);
                for (int nb = 0; nb < NB; ++nb)
                    tma_load_3d(q_s + nb * BM * 128, &map_q, q_full, nb * 64, kvh * G, q0 + tok_first);
            }
            // Keys and values have cursors of their own: a key tile's place is free as soon as its
            // scores are formed, which is before the product with the values of the tile before it.
            bool ok = true;
            int armed_k = 0, armed_v = 0;
            long long t_idle = -1;
            auto row_of = [&](int j) {
                const int posn = (t_lo + j) * BN;
                const int page = p.table[(long long)seq * p.pages_per_seq + (posn % p.ring) / BN];
                return (page * p.nkv + kvh) * BN;
            };
            while (armed_v < n_tiles && ok) {
                bool moved = false;
                if (armed_k < n_tiles) {
                    const int j = armed_k, s = j % KV_STAGES;
                    if (mbar_test_wait(&k_empty[s], (uint32_t)(((j / KV_STAGES) & 1) ^ 1))) {
                        const int row = row_of(j);
                        mbar_expect_tx(&k_full[s], KV_BYTES);
                        for (int nb = 0; nb < NB; ++nb) tma_load_2d(k_s + s * KV_BYTES + nb * BN * 128, &map_k, &k_full[s], nb * 64, row);
                        armed_k = j + 1;
                        moved = true;
                    }
                }
                if (armed_v < armed_k) {
                    const int j = armed_v, s = j % KV_STAGES;
                    if (mbar_test_wait(&v_empty[s], (uint32_t)(((j / KV_STAGES) & 1) ^ 1))) {
                        const int row = row_of(j);
                        mbar_expect_tx(&v_full[s], KV_BYTES);
                        for (int nb = 0; nb < NB; ++nb) tma_load_2d(v_s + s * KV_BYTES + nb * BN * 128, &map_v, &v_full[s], nb * 64, row);
                        armed_v = j + 1;
                        moved = true;
                    }
                }
                if (moved) { t_idle = -1; continue; }
                if (*err) { ok = false; break; }
                if (t_idle < 0) t_idle = clock64();
                else if (clock64() - t_idle > WAIT_LIMIT_CYCLES) { *err = 1; ok = false; }
            }
            if (*err) {          // let the copies in flight land before the CTA's memory goes away
                const long long tstart = clock64();
                while (n_tiles > 0 && !mbar_try_wait(q_full, 0)) if (clock64() - tstart > WAIT_LIMIT_CYCLES / 8) break;
                for (int j = max(0, armed_k - KV_STAGES); j < armed_k; ++j)
                    while (!mbar_try_wait(&k_full[j % KV_STAGES], (j / KV_STAGES) & 1)) if (clock64() - tstart > WAIT_LIMIT_CYCLES / 4) break;
                for (int j = max(0, armed_v - KV_STAGES); j < armed_v; ++j)
                    while (!mbar_try_wait(&v_full[j % KV_STAGES], (j / KV_STAGES) & 1)) if (clock64() - tstart > WAIT_LIMIT_CYCLES / 4) break;
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA ----------------
        if (lane == 0) {
            // Every descriptor is a constant away from three made once: the address field counts 16-byte
            // units and shared memory ends far below where it would carry into the next field.
            constexpr uint32_t idesc_qk = idesc_bf16(BM, BN, 0);
            constexpr uint32_t idesc_pv = idesc_bf16(BM, HD, 1);          // all HD output columns in one MMA
            const uint64_t q_desc = make_desc(smem_u32(q_s));
            const uint64_t k_desc = make_desc(smem_u32(k_s));
            const uint64_t v_desc = make_desc_mn(smem_u32(v_s));
            auto issue_qk = [&](int j) {
                const int s = j % KV_STAGES;
                const uint64_t kd = k_desc + (uint64_t)(s * (KV_BYTES >> 4));
                const uint32_t acc = tmem_base + (uint32_t)((j & 1) * BN);
#pragma unroll
                for (int ks = 0; ks < HD / 16; ++ks) {
                    const uint64_t da = q_desc + (uint64_t)(((ks / 4) * BM * 128 + (ks % 4) * 32) >> 4);
                    const uint64_t db = kd + (uint64_t)(((ks / 4) * BN * 128 + (ks % 4) * 32) >> 4);
                    tc_mma_bf16(acc, da, db, idesc_qk, ks > 0 ? 1u : 0u);
                }
                tc_commit(&s_full[j & 1]);
                tc_commit(&k_empty[s]);
            };
            // MMAs run in the order of their issue: the scores of tile j+1 may be queued over the place
            // of tile j-1's probabilities as soon as the product that reads those has been issued.
            bool ok = n_tiles > 0 ? mbar_wait(q_full, 0, err) : true;
            if (ok && n_tiles > 0) ok = mbar_wait(&k_full[0], 0, err);
            if (ok && n_tiles > 0) { tc_fence_after(); issue_qk(0); }
            for (int j = 0; j < n_tiles && ok; ++j) {
                if (j + 1 < n_tiles) {
                    ok = mbar_wait(&k_full[(j + 1) % KV_STAGES], (uint32_t)(((j + 1) / KV_STAGES) & 1), err);
                    if (!ok) break;
                    tc_fence_after();
                    issue_qk(j + 1);
                }
                ok = mbar_wait(&p_full[j & 1], (uint32_t)((j >> 1) & 1), err);
                if (ok) ok = mbar_wait(&v_full[j % KV_STAGES], (uint32_t)((j / KV_STAGES) & 1), err);
                if (!ok) break;
                tc_fence_after();
                const uint64_t vd = v_desc + (uint64_t)((j % KV_STAGES) * (KV_BYTES >> 4));
                const uint32_t p_t = tmem_base + (uint32_t)((j & 1) * BN);
#pragma unroll
                for (int ks = 0; ks < BN / 16; ++ks)
                    tc_mma_bf16_ts(tmem_base + O_COL, p_t + ks * 8, vd + (uint64_t)((ks * 16 * 128) >> 4), idesc_pv,
                                   (j > 0 || ks > 0) ? 1u : 0u);
                tc_commit(&pv_done[j & 1]);
                tc_commit(&v_empty[j % KV_STAGES]);
            }
        }
    } else {
        // ---------------- softmax: one thread a row ----------------
        const int q = warp & 3;
        const int r = q * 32 + lane;                       // row of the tile = lane of tensor memory
        const int tok = tok_first + r / G, g = r % G;
        const bool row_ok = r < TPB * G && tok < q_len;
        const int row_pos = before + tok;
        const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
        const int st = (warp - 2) * 32 + lane;             // 0..127 among the softmax threads
        float m_ref = -INFINITY, l = 0.f;
        bool ok = true;
        for (int j = 0; j < n_tiles && ok; ++j) {
            const int b = j & 1;
            const int base = (t_lo + j) * BN;
            if (base + BN - 1 > last_pos) {
                // rows of V past the sequence's end hold whatever the page held before: make them zero
                ok = mbar_wait(&v_full[j % KV_STAGES], (uint32_t)((j / KV_STAGES) & 1), err);
                if (!ok) break;
                const int first = last_pos + 1 - base;     // first row to clear (>= 1: the tile holds a valid key)
                uint8_t* vt = v_s + (j % KV_STAGES) * KV_BYTES;
                for (int i = st; i < (BN - first) * NB * 8; i += 128) {
                    const int row = first + i / (NB * 8), rest = i % (NB * 8);
                    *reinterpret_cast<uint4*>(vt + (rest / 8) * BN * 128 + row * 128 + (rest % 8) * 16) = make_uint4(0, 0, 0, 0);
                }
                fence_proxy_async();
            }
            ok = mbar_wait(&s_full[b], (uint32_t)((j >> 1) & 1), err);
            if (!ok) break;
            tc_fence_after();
            uint32_t raw[BN];
            tmem_ld32(lane_addr + (uint32_t)(b * BN), raw);
            tmem_ld32(lane_addr + (uint32_t)(b * BN + 32), raw + 32);
            tmem_ld_wait();
            // scores stay raw (q.k); the scale goes into the exponent: p = 2^(s c - m).  A tile that
            // every row of the CTA sees whole needs no mask.
            const bool whole = row_ok && base + BN - 1 <= before + tok_first && p.window <= 0 && r < TPB * G;
            if (!__all_sync(0xffffffffu, whole)) {
#pragma unroll
                for (int cI = 0; cI < BN; ++cI) {
                    const int kp = base + cI;
                    const bool vis = row_ok && kp <= row_pos && (p.window <= 0 || kp > row_pos - p.window);
                    if (!vis) raw[cI] = __float_as_uint(-INFINITY);
                }
            }
            float mxs[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};   // four chains of three-input maxima
#pragma unroll
            for (int cI = 0; cI < BN; cI += 8)
#pragma unroll
                for (int ch = 0; ch < 4; ++ch)
                    mxs[ch] = max3(mxs[ch], __uint_as_float(raw[cI + 2 * ch]), __uint_as_float(raw[cI + 2 * ch + 1]));
            float mx = fmaxf(fmaxf(mxs[0], mxs[1]), fmaxf(mxs[2], mxs[3]));
            mx *= p.c;                                       // c > 0: the maximum in exponent units
            // raise the reference maximum only when it lags by more than RESCALE_STEP (or is not set)
            const bool grow = mx > m_ref + RESCALE_STEP || (m_ref == -INFINITY && mx > -INFINITY);
            if (__any_sync(0xffffffffu, grow)) {
                const float m_new = grow ? mx : m_ref;
                const float f = (m_ref == -INFINITY || !grow) ? (grow ? 0.f : 1.f) : exp2f(m_ref - m_new);
                if (j > 0) {
                    ok = mbar_wait(&pv_done[(j - 1) & 1], (uint32_t)(((j - 1) >> 1) & 1), err);   // O is at rest
                    if (!ok) break;
                    tc_fence_after();
#pragma unroll
                    for (int cb = 0; cb < HD / 32; ++cb) {
                        uint32_t oo[32];
                        tmem_ld32(lane_addr + (uint32_t)(O_COL + cb * 32), oo);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 32; ++i) oo[i] = __float_as_uint(__uint_as_float(oo[i]) * f);
                        tmem_st32(lane_addr + (uint32_t)(O_COL + cb * 32), oo);
                    }
                    tmem_st_wait();
                }
                l *= f;
                m_ref = m_new;
            }
            const float mb = m_ref == -INFINITY ? 0.f : m_ref;
            uint32_t packed[BN / 2];
            const uint64_t c2 = pair_of(p.c, p.c), shift2 = pair_of(-mb, -mb);
            uint64_t sums[2] = {pair_of(0.f, 0.f), pair_of(0.f, 0.f)};
#pragma unroll
            for (int cI = 0; cI < BN; cI += 2) {
                float x0, x1;
                halves_of(fma_pair(pair_of(__uint_as_float(raw[cI]), __uint_as_float(raw[cI + 1])), c2, shift2), x0, x1);
                const float p0 = ex2(x0), p1 = ex2(x1);
                sums[(cI >> 1) & 1] = add_pair(sums[(cI >> 1) & 1], pair_of(p0, p1));
                __nv_bfloat162 pr = __floats2bfloat162_rn(p0, p1);
                packed[cI / 2] = *reinterpret_cast<uint32_t*>(&pr);
            }
            float s0, s1, s2, s3;
            halves_of(sums[0], s0, s1);
            halves_of(sums[1], s2, s3);
            l += (s0 + s1) + (s2 + s3);
            tmem_st32(lane_addr + (uint32_t)(b * BN), packed);
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&p_full[b]);         // one arrival a warp
        }
        if (ok && n_tiles > 0) ok = mbar_wait(&pv_done[(n_tiles - 1) & 1], (uint32_t)(((n_tiles - 1) >> 1) & 1), err);
        if (ok) {
            tc_fence_after();
            const bool partial = DECODE && p.n_slices > 1;
            const float inv = partial ? 1.0f : (l > 0.f ? 1.0f / l : 0.f);
            const int head = kvh * G + g;
            bf16* dst = p.out + (long long)(q0 + tok) * p.o_stride + (long long)head * HD;
            const long long pi = partial ? ((long long)seq * p.nh + head) * p.n_slices + blockIdx.x : 0;
            if (partial && row_ok) { p.part_ml[pi * 2] = m_ref; p.part_ml[pi * 2 + 1] = l; }
#pragma unroll
            for (int cb = 0; cb < HD / 32; ++cb) {
                uint32_t oo[32];
                if (n_tiles > 0) {
                    tmem_ld32(lane_addr + (uint32_t)(O_COL + cb * 32), oo);
                    tmem_ld_wait();
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) oo[i] = 0;
                }
                if (row_ok && partial) {
#pragma unroll
                    for (int i = 0; i < 32; i += 4)
                        *reinterpret_cast<uint4*>(p.part_o + pi * HD + cb * 32 + i) = make_uint4(oo[i], oo[i + 1], oo[i + 2], oo[i + 3]);
                } else if (row_ok) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        uint4 w;
                        __nv_bfloat162 a0 = __floats2bfloat162_rn(__uint_as_float(oo[i]) * inv, __uint_as_float(oo[i + 1]) * inv);
                        __nv_bfloat162 a1 = __floats2bfloat162_rn(__uint_as_float(oo[i + 2]) * inv, __uint_as_float(oo[i + 3]) * inv);
                        __nv_bfloat162 a2 = __floats2bfloat162_rn(__uint_as_float(oo[i + 4]) * inv, __uint_as_float(oo[i + 5]) * inv);
                        __nv_bfloat162 a3 = __floats2bfloat162_rn(__uint_as_float(oo[i + 6]) * inv, __uint_as_float(oo[i + 7]) * inv);
                        w.x = *reinterpret_cast<uint32_t*>(&a0); w.y = *reinterpret_cast<uint32_t*>(&a1);
                        w.z = *reinterpret_cast<uint32_t*>(&a2); w.w = *reinterpret_cast<uint32_t*>(&a3);
                        *reinterpret_cast<uint4*>(dst + cb * 32 + i) = w;
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
    if (threadIdx.x == 0 && *err) atomicExch(p.error, 1);
}

// ---------------------------------------------------------------------------------------
// Prompts, 256 rows a CTA: two query tiles of 128 rows share every key and value tile, so a tile is
// fetched from the L2 and written to shared memory once for both, and five such tiles can be in
// flight.  One CTA an SM with all of its tensor memory: tile t has its scores in columns
// [128 t, 128 t + 128) (two buffers) and its output in [256 + 128 t, ...).  Warp 0 issues TMA,
// warps 1 and 2 issue one tile's MMAs each (MMAs of one thread run in the order of their issue, which
// is what lets a tile's next scores be queued behind the product that reads the buffer they fall
// into), warps 4-7 and 8-11 are the two tiles' softmax.  A key tile's place is given back when both
// issuers have let go of it; an issuer whose rows do not see a tile lets go of it at once.
constexpr int WIDE_TILES = 2;
constexpr int WIDE_STAGES = HD == 128 ? 4 : 8;
constexpr int WIDE_THREADS = 384;
constexpr int WIDE_TMEM = 512;
constexpr int WIDE_O_COL = 256;
constexpr int WIDE_MIN_BLOCKS = 148;         // fewer blocks than SMs: the kernel of 128 rows a CTA spreads the work further
constexpr int wide_smem_bytes() { return WIDE_TILES * Q_BYTES + 2 * WIDE_STAGES * KV_BYTES + 1024 + 512; }

__global__ void __launch_bounds__(WIDE_THREADS, 1)
attn_tc_wide_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                    const __grid_constant__ CUtensorMap map_v, TcAttnParams p) {
    extern __shared__ uint8_t smem_raw[];
    constexpr int S = WIDE_STAGES;
    const int per_tile = p.n_seqs * p.nkv;
    const int seq = (blockIdx.x % per_tile) / p.nkv;
    const int kvh = blockIdx.x % p.nkv;
    const int q0 = p.seq_start[seq], q_len = p.seq_start[seq + 1] - q0, before = p.seq_before[seq];
    const int G = p.group;
    const int TPB = BM / G;                                // tokens a query tile
    const int wide_tile = p.n_row_tiles - 1 - blockIdx.x / per_tile;     // longest first
    const int tok_first = wide_tile * WIDE_TILES * TPB;
    if (tok_first >= q_len) return;

    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* q_s = smem;
    uint8_t* k_s = q_s + WIDE_TILES * Q_BYTES;
    uint8_t* v_s = k_s + S * KV_BYTES;
    uint64_t* bars = (uint64_t*)(v_s + S * KV_BYTES);
    uint64_t* q_full = bars;                               // [2]
    uint64_t* k_full = q_full + WIDE_TILES;
    uint64_t* k_empty = k_full + S;
    uint64_t* v_full = k_empty + S;
    uint64_t* v_empty = v_full + S;
    uint64_t* s_full = v_empty + S;                        // [tile][2]
    uint64_t* p_full = s_full + 2 * WIDE_TILES;
    uint64_t* pv_done = p_full + 2 * WIDE_TILES;
    uint32_t* tmem_slot = (uint32_t*)(pv_done + 2 * WIDE_TILES);
    volatile int* err = (volatile int*)(tmem_slot + 1);
    static_assert((WIDE_TILES + 4 * WIDE_STAGES + 6 * WIDE_TILES) * 8 + 8 <= 512, "barriers outgrew their place");

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int last_pos = before + q_len - 1;
    // what each query tile sees: tiles [lo, hi] of the sequence's keys; the CTA walks their union
    int lo[WIDE_TILES], hi[WIDE_TILES], tokf[WIDE_TILES];
    bool has[WIDE_TILES];
#pragma unroll
    for (int t = 0; t < WIDE_TILES; ++t) {
        tokf[t] = tok_first + t * TPB;
        has[t] = tokf[t] < q_len;
        const int tokl = min(q_len - 1, tokf[t] + TPB - 1);
        hi[t] = (before + tokl) / BN;
        lo[t] = p.window > 0 ? max(0, before + tokf[t] - p.window + 1) / BN : 0;
    }
    const int t_lo = lo[0];
    const int t_hi = has[1] ? hi[1] : hi[0];
    const int n_union = t_hi - t_lo + 1;

    if (threadIdx.x == 0) {
        for (int t = 0; t < WIDE_TILES; ++t) mbar_init(&q_full[t], 1);
        for (int s = 0; s < S; ++s) {
            mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], WIDE_TILES);
            mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], WIDE_TILES);
        }
        for (int b = 0; b < 2 * WIDE_TILES; ++b) { mbar_init(&s_full[b], 1); mbar_init(&p_full[b], 4); mbar_init(&pv_done[b], 1); }
        *err = 0;
        fence_barrier_init();
    }
    if (warp == 1) { tmem_alloc(tmem_slot, WIDE_TMEM); tmem_relinquish(); }
    if (warp == 0 && lane == 0) { prefetch_tmap(&map_q); prefetch_tmap(&map_k); prefetch_tmap(&map_v); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_trigger();                                         // after the allocation, as in attn_tc_kernel
    pdl_wait();

    if (warp == 0) {
        // ---------------- TMA ----------------
        if (lane == 0) {
#pragma unroll
            for (int t = 0; t < WIDE_TILES; ++t)
                if (has[t]) {
                    mbar_expect_tx(&q_full[t], NB * TPB * G * 128);
                    for (int nb = 0; nb < NB; ++nb)
                        tma_load_3d(q_s + t * Q_BYTES + nb * BM * 128, &map_q, &q_full[t], nb * 64, kvh * G, q0 + tokf[t]);
                }
            bool ok = true;
            int armed_k = 0, armed_v = 0;
            long long t_idle = -1;
            auto row_of = [&](int j) {
                const int posn = (t_lo + j) * BN;
                const int page = p.table[(long long)seq * p.pages_per_seq + (posn % p.ring) / BN];
                return (page * p.nkv + kvh) * BN;
            };
            while (armed_v < n_union && ok) {
                bool moved = false;
                if (armed_k < n_union) {
                    const int j = armed_k, s = j % S;
                    if (mbar_test_wait(&k_empty[s], (uint32_t)(((j / S) & 1) ^ 1))) {
                        const int row = row_of(j);
                        mbar_expect_tx(&k_full[s], KV_BYTES);
                        for (int nb = 0; nb < NB; ++nb) tma_load_2d(k_s + s * KV_BYTES + nb * BN * 128, &map_k, &k_full[s], nb * 64, row);
                        armed_k = j + 1;
                        moved = true;
                    }
                }
                if (armed_v < armed_k) {
                    const int j = armed_v, s = j % S;
                    if (mbar_test_wait(&v_empty[s], (uint32_t)(((j / S) & 1) ^ 1))) {
                        const int row = row_of(j);
                        mbar_expect_tx(&v_full[s], KV_BYTES);
                        for (int nb = 0; nb < NB; ++nb) tma_load_2d(v_s + s * KV_BYTES + nb * BN * 128, &map_v, &v_full[s], nb * 64, row);
                        armed_v = j + 1;
                        moved = true;
                    }
                }
                if (moved) { t_idle = -1; continue; }
                if (*err) { ok = false; break; }
                if (t_idle < 0) t_idle = clock64();
                else if (clock64() - t_idle > WAIT_LIMIT_CYCLES) { *err = 1; ok = false; }
            }
            if (*err) {          // let the copies in flight land before the CTA's memory goes away
                const long long tstart = clock64();
                for (int t = 0; t < WIDE_TILES; ++t)
                    while (has[t] && !mbar_try_wait(&q_full[t], 0)) if (clock64() - tstart > WAIT_LIMIT_CYCLES / 8) break;
                for (int j = max(0, armed_k - S); j < armed_k; ++j)
                    while (!mbar_try_wait(&k_full[j % S], (j / S) & 1)) if (clock64() - tstart > WAIT_LIMIT_CYCLES / 4) break;
                for (int j = max(0, armed_v - S); j < armed_v; ++j)
                    while (!mbar_try_wait(&v_full[j % S], (j / S) & 1)) if (clock64() - tstart > WAIT_LIMIT_CYCLES / 4) break;
            }
        }
    } else if (warp == 1 || warp == 2) {
        // ---------------- MMA, one query tile a warp ----------------
        if (lane == 0) {
            const int t = warp - 1;
            const int first = has[t] ? lo[t] - t_lo : 0;
            const int n_act = has[t] ? hi[t] - lo[t] + 1 : 0;
            constexpr uint32_t idesc_qk = idesc_bf16(BM, BN, 0);
            constexpr uint32_t idesc_pv = idesc_bf16(BM, HD, 1);
            const uint64_t q_desc = make_desc(smem_u32(q_s + t * Q_BYTES));
            const uint64_t k_desc = make_desc(smem_u32(k_s));
            const uint64_t v_desc = make_desc_mn(smem_u32(v_s));
            const uint32_t s_base = tmem_base + (uint32_t)(t * 2 * BN);
            const uint32_t o_base = tmem_base + (uint32_t)(WIDE_O_COL + t * HD);
            uint64_t* sf = s_full + 2 * t;
            uint64_t* pf = p_full + 2 * t;
            uint64_t* pd = pv_done + 2 * t;
            bool ok = true;
            // a tile of keys these rows do not see: wait until it is there (which keeps this thread's
            // arrivals in step with the loads), then give its place back
            auto pass_by = [&](int j) {
                const int s = j % S;
                const uint32_t ph = (uint32_t)((j / S) & 1);
                ok = mbar_wait(&k_full[s], ph, err);
                if (!ok) return;
                mbar_arrive(&k_empty[s]);
                ok = mbar_wait(&v_full[s], ph, err);
                if (!ok) return;
                mbar_arrive(&v_empty[s]);
            };
            auto issue_qk = [&](int i) {                   // i counts this tile's own key tiles
                const int j = first + i, s = j % S;
                const uint64_t kd = k_desc + (uint64_t)(s * (KV_BYTES >> 4));
                const uint32_t acc = s_base + (uint32_t)((i & 1) * BN);
#pragma unroll
                for (int ks = 0; ks < HD / 16; ++ks) {
                    const uint64_t da = q_desc + (uint64_t)(((ks / 4) * BM * 128 + (ks % 4) * 32) >> 4);
                    const uint64_t db = kd + (uint64_t)(((ks / 4) * BN * 128 + (ks % 4) * 32) >> 4);
                    tc_mma_bf16(acc, da, db, idesc_qk, ks > 0 ? 1u : 0u);
                }
                tc_commit(&sf[i & 1]);
                tc_commit(&k_empty[s]);
            };
            for (int j = 0; j < first && ok; ++j) pass_by(j);
            if (ok && n_act > 0) ok = mbar_wait(&q_full[t], 0, err);
            if (ok && n_act > 0) ok = mbar_wait(&k_full[first % S], (uint32_t)((first / S) & 1), err);
            if (ok && n_act > 0) { tc_fence_after(); issue_qk(0); }
            for (int i = 0; i < n_act && ok; ++i) {
                const int j = first + i;
                if (i + 1 < n_act) {
                    ok = mbar_wait(&k_full[(j + 1) % S], (uint32_t)(((j + 1) / S) & 1), err);
                    if (!ok) break;
                    tc_fence_after();
                    issue_qk(i + 1);
                }
                ok = mbar_wait(&pf[i & 1], (uint32_t)((i >> 1) & 1), err);
                if (ok) ok = mbar_wait(&v_full[j % S], (uint32_t)((j / S) & 1), err);
                if (!ok) break;
                tc_fence_after();
                const uint64_t vd = v_desc + (uint64_t)((j % S) * (KV_BYTES >> 4));
                const uint32_t p_t = s_base + (uint32_t)((i & 1) * BN);
#pragma unroll
                for (int ks = 0; ks < BN / 16; ++ks)
                    tc_mma_bf16_ts(o_base, p_t + ks * 8, vd + (uint64_t)((ks * 16 * 128) >> 4), idesc_pv, (i > 0 || ks > 0) ? 1u : 0u);
                tc_commit(&pd[i & 1]);
                tc_commit(&v_empty[j % S]);
            }
            for (int j = first + n_act; j < n_union && ok; ++j) pass_by(j);
        }
    } else if (warp >= 4) {
        // ---------------- softmax: one thread a row, four warps a query tile ----------------
        const int t = (warp - 4) >> 2;
        const int q = warp & 3;
        const int r = q * 32 + lane;                       // row of the tile = lane of tensor memory
        const int tok = tokf[t] + r / G, g = r % G;
        const bool row_ok = has[t] && r < TPB * G && tok < q_len;
        const int row_pos = before + tok;
        const int first = has[t] ? lo[t] - t_lo : 0;
        const int n_act = has[t] ? hi[t] - lo[t] + 1 : 0;
        const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
        const uint32_t s_base = lane_addr + (uint32_t)(t * 2 * BN);
        const uint32_t o_base = lane_addr + (uint32_t)(WIDE_O_COL + t * HD);
        uint64_t* sf = s_full + 2 * t;
        uint64_t* pf = p_full + 2 * t;
        uint64_t* pd = pv_done + 2 * t;
        const int st = (warp & 3) * 32 + lane;             // 0..127 among the tile's softmax threads
        float m_ref = -INFINITY, l = 0.f;
        bool ok = true;
        for (int i = 0; i < n_act && ok; ++i) {
            const int b = i & 1;
            const int j = first + i;
            const int base = (t_lo + j) * BN;
            if (base + BN - 1 > last_pos) {
                // rows of V past the sequence's end hold whatever the page held before: make them zero
                // (both query tiles do, before their own products with this tile)
                ok = mbar_wait(&v_full[j % S], (uint32_t)((j / S) & 1), err);
                if (!ok) break;
                const int zfirst = last_pos + 1 - base;    // first row to clear (>= 1: the tile holds a valid key)
                uint8_t* vt = v_s + (j % S) * KV_BYTES;
                for (int x = st; x < (BN - zfirst) * NB * 8; x += 128) {
                    const int row = zfirst + x / (NB * 8), rest = x % (NB * 8);
                    *reinterpret_cast<uint4*>(vt + (rest / 8) * BN * 128 + row * 128 + (rest % 8) * 16) = make_uint4(0, 0, 0, 0);
                }
                fence_proxy_async();
            }
            ok = mbar_wait(&sf[b], (uint32_t)((i >> 1) & 1), err);
            if (!ok) break;
            tc_fence_after();
            uint32_t raw[BN];
            tmem_ld32(s_base + (uint32_t)(b * BN), raw);
            tmem_ld32(s_base + (uint32_t)(b * BN + 32), raw + 32);
            tmem_ld_wait();
            const bool whole = row_ok && base + BN - 1 <= before + tokf[t] && p.window <= 0;
            if (!__all_sync(0xffffffffu, whole)) {
#pragma unroll
                for (int cI = 0; cI < BN; ++cI) {
                    const int kp = base + cI;
                    const bool vis = row_ok && kp <= row_pos && (p.window <= 0 || kp > row_pos - p.window);
                    if (!vis) raw[cI] = __float_as_uint(-INFINITY);
                }
            }
            float mxs[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int cI = 0; cI < BN; cI += 8)
#pragma unroll
                for (int ch = 0; ch < 4; ++ch)
                    mxs[ch] = max3(mxs[ch], __uint_as_float(raw[cI + 2 * ch]), __uint_as_float(raw[cI + 2 * ch + 1]));
            float mx = fmaxf(fmaxf(mxs[0], mxs[1]), fmaxf(mxs[2], mxs[3]));
            mx *= p.c;
            const bool grow = mx > m_ref + RESCALE_STEP || (m_ref == -INFINITY && mx > -INFINITY);
            if (__any_sync(0xffffffffu, grow)) {
                const float m_new = grow ? mx : m_ref;
                const float f = (m_ref == -INFINITY || !grow) ? (grow ? 0.f : 1.f) : exp2f(m_ref - m_new);
                if (i > 0) {
                    ok = mbar_wait(&pd[(i - 1) & 1], (uint32_t)(((i - 1) >> 1) & 1), err);   // O is at rest
                    if (!ok) break;
                    tc_fence_after();
#pragma unroll
                    for (int cb = 0; cb < HD / 32; ++cb) {
                        uint32_t oo[32];
                        tmem_ld32(o_base + (uint32_t)(cb * 32), oo);
                        tmem_ld_wait();
#pragma unroll
                        for (int x = 0; x < 32; ++x) oo[x] = __float_as_uint(__uint_as_float(oo[x]) * f);
                        tmem_st32(o_base + (uint32_t)(cb * 32), oo);
                    }
                    tmem_st_wait();
                }
                l *= f;
                m_ref = m_new;
            }
            const float mb = m_ref == -INFINITY ? 0.f : m_ref;
            uint32_t packed[BN / 2];
            const uint64_t c2 = pair_of(p.c, p.c), shift2 = pair_of(-mb, -mb);
            uint64_t sums[2] = {pair_of(0.f, 0.f), pair_of(0.f, 0.f)};
#pragma unroll
            for (int cI = 0; cI < BN; cI += 2) {
                float x0, x1;
                halves_of(fma_pair(pair_of(__uint_as_float(raw[cI]), __uint_as_float(raw[cI + 1])), c2, shift2), x0, x1);
                const float p0 = ex2(x0), p1 = ex2(x1);
                sums[(cI >> 1) & 1] = add_pair(sums[(cI >> 1) & 1], pair_of(p0, p1));
                __nv_bfloat162 pr = __floats2bfloat162_rn(p0, p1);
                packed[cI / 2] = *reinterpret_cast<uint32_t*>(&pr);
            }
            float s0, s1, s2, s3;
            halves_of(sums[0], s0, s1);
            halves_of(sums[1], s2, s3);
            l += (s0 + s1) + (s2 + s3);
            tmem_st32(s_base + (uint32_t)(b * BN), packed);
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&pf[b]);
        }
        if (ok && n_act > 0) ok = mbar_wait(&pd[(n_act - 1) & 1], (uint32_t)(((n_act - 1) >> 1) & 1), err);
        if (ok && n_act > 0) {
            tc_fence_after();
            const float inv = l > 0.f ? 1.0f / l : 0.f;
            const int head = kvh * G + g;
            bf16* dst = p.out + (long long)(q0 + tok) * p.o_stride + (long long)head * HD;
#pragma unroll
            for (int cb = 0; cb < HD / 32; ++cb) {
                uint32_t oo[32];
                tmem_ld32(o_base + (uint32_t)(cb * 32), oo);
                tmem_ld_wait();
                if (row_ok) {
#pragma unroll
                    for (int x = 0; x < 32; x += 8) {
                        uint4 w;
                        __nv_bfloat162 a0 = __floats2bfloat162_rn(__uint_as_float(oo[x]) * inv, __uint_as_float(oo[x + 1]) * inv);
                        __nv_bfloat162 a1 = __floats2bfloat162_rn(__uint_as_float(oo[x + 2]) * inv, __uint_as_float(oo[x + 3]) * inv);
                        __nv_bfloat162 a2 = __floats2bfloat162_rn(__uint_as_float(oo[x + 4]) * inv, __uint_as_float(oo[x + 5]) * inv);
                        __nv_bfloat162 a3 = __floats2bfloat162_rn(__uint_as_float(oo[x + 6]) * inv, __uint_as_float(oo[x + 7]) * inv);
                        w.x = *reinterpret_cast<uint32_t*>(&a0); w.y = *reinterpret_cast<uint32_t*>(&a1);
                        w.z = *reinterpret_cast<uint32_t*>(&a2); w.w = *reinterpret_cast<uint32_t*>(&a3);
                        *reinterpret_cast<uint4*>(dst + cb * 32 + x) = w;
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, WIDE_TMEM);
    }
    if (threadIdx.x == 0 && *err) atomicExch(p.error, 1);
}

// ---------------------------------------------------------------------------------------
UB_API int ub_attn_tc_head_dim() { return HD; }

// tensor map of q as [tokens, heads, HD] (row stride q_stride elements), boxes of 64 x group x floor(128/group)
UB_API int ub_attn_tc_map_q(void* out_map, const void* q, long long n_tokens, int nh, long long q_stride, int group) {
    EncodeTiledFn enc = tensor_map_encoder();
    if (!enc) return UB_ERR_UNSUPPORTED;
    if (((uintptr_t)q & 15) || (q_stride * 2) % 16 != 0 || group < 1 || group > BM || n_tokens < 1) return UB_ERR_ARG;
    cuuint64_t dims[3] = {(cuuint64_t)HD, (cuuint64_t)nh, (cuuint64_t)n_tokens};
    cuuint64_t strides[2] = {(cuuint64_t)HD * 2, (cuuint64_t)q_stride * 2};
    cuuint32_t box[3] = {64, (cuuint32_t)group, (cuuint32_t)(BM / group)};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = enc((CUtensorMap*)out_map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, (void*)q, dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : UB_ERR_ARG;
}
// tensor map of one run's K or V cache [pages, kv heads, 64, HD] as rows of HD, boxes of 64 x 64
UB_API int ub_attn_tc_map_kv(void* out_map, const void* cache, long long n_pages, int nkv) {
    EncodeTiledFn enc = tensor_map_encoder();
    if (!enc) return UB_ERR_UNSUPPORTED;
    if (((uintptr_t)cache & 15) || n_pages < 1) return UB_ERR_ARG;
    cuuint64_t dims[2] = {(cuuint64_t)HD, (cuuint64_t)(n_pages * nkv * BN)};
    cuuint64_t strides[1] = {(cuuint64_t)HD * 2};
    cuuint32_t box[2] = {64, (cuuint32_t)BN};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc((CUtensorMap*)out_map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (void*)cache, dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : UB_ERR_ARG;
}

// merge the slices of a decode step: grid (sequences * heads), HD threads
__global__ void attn_tc_combine_kernel(TcAttnParams p) {
    pdl_trigger();
    pdl_wait();
    const int sh = blockIdx.x, d = threadIdx.x;
    const int seq = sh / p.nh, head = sh % p.nh;
    const long long base = (long long)sh * p.n_slices;
    float mm = -INFINITY;
    for (int s = 0; s < p.n_slices; ++s) mm = fmaxf(mm, p.part_ml[(base + s) * 2]);
    float acc = 0.f, ll = 0.f;
    for (int s = 0; s < p.n_slices; ++s) {
        const float ms = p.part_ml[(base + s) * 2];
        const float f = ms == -INFINITY ? 0.f : exp2f(ms - mm);
        ll += f * p.part_ml[(base + s) * 2 + 1];
        acc += f * p.part_o[(base + s) * HD + d];
    }
    p.out[(long long)p.seq_start[seq] * p.o_stride + (long long)head * HD + d] = __float2bfloat16_rn(acc / ll);
}

template <int STAGES, bool DECODE>
static int launch_attn(dim3 grid, const void* map_q, const void* map_k, const void* map_v, const TcAttnParams& p, cudaStream_t st) {
    static bool attr_done = false;
    auto kern = attn_tc_kernel<STAGES, DECODE>;
    if (!attr_done) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes(STAGES));
        if (e != cudaSuccess) return (int)e;
        attr_done = true;
    }
    cudaError_t e = ub_launch_dependent(kern, grid, dim3(NTHREADS), (size_t)smem_bytes(STAGES), st,
                                        *(const CUtensorMap*)map_q, *(const CUtensorMap*)map_k, *(const CUtensorMap*)map_v, p);
    return (int)e;
}

static int g_wide = 1;
// 1 (the default): prompts take the kernel of 256 rows a CTA when that gives every SM a CTA; 0: never; 2: always
UB_API void ub_attn_tc_set_wide(int on) { g_wide = on; }

static int launch_wide(unsigned blocks, const void* map_q, const void* map_k, const void* map_v, const TcAttnParams& p, cudaStream_t st) {
    static bool attr_done = false;
    if (!attr_done) {
        cudaError_t e = cudaFuncSetAttribute(attn_tc_wide_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, wide_smem_bytes());
        if (e != cudaSuccess) return (int)e;
        attr_done = true;
    }
    return (int)ub_launch_dependent(attn_tc_wide_kernel, dim3(blocks), dim3(WIDE_THREADS), (size_t)wide_smem_bytes(), st,
                                    *(const CUtensorMap*)map_q, *(const CUtensorMap*)map_k, *(const CUtensorMap*)map_v, p);
}

// mode 0: prompts (any numbers of new tokens); mode 1: one new token a sequence, keys in n_slices slices
// (part_o: float32 [n_seqs, nh, n_slices, HD], part_ml: [.., 2] when n_slices > 1).
UB_API int ub_attn_tc(int mode, const void* map_q, const void* map_k, const void* map_v, void* out, long long o_stride,
                      const int* seq_start, const int* seq_before, const int* table, int pages_per_seq,
                      int ring, int page, int n_seqs, int max_new, int nh, int nkv, int window, float scale,
                      int n_slices, float* part_o, float* part_ml, int* error, cudaStream_t st) {
    if (n_seqs <= 0 || max_new <= 0) return 0;
    const int group = nh / nkv;
    if (page != BN || ring % page != 0 || nh % nkv != 0 || group > BM || (o_stride % 8) != 0 || ((uintptr_t)out & 15))
        return UB_ERR_ARG;
    if (n_seqs > 65535 || nkv > 65535) return UB_ERR_ARG;
    TcAttnParams p;
    p.out = (bf16*)out; p.o_stride = o_stride; p.seq_start = seq_start; p.seq_before = seq_before; p.table = table;
    p.pages_per_seq = pages_per_seq; p.ring = ring; p.nkv = nkv; p.group = group; p.window = window;
    p.c = scale * 1.4426950408889634f; p.error = error;
    p.part_o = part_o; p.part_ml = part_ml; p.n_slices = n_slices < 1 ? 1 : n_slices; p.nh = nh;
    p.n_seqs = n_seqs; p.n_row_tiles = 1;
    if (mode == 0) {
        p.n_slices = 1;
        const int tpb = BM / group;
        p.n_seqs = n_seqs;
        const long long wide_tiles = (max_new + WIDE_TILES * tpb - 1) / (WIDE_TILES * tpb);
        const long long wide_blocks = wide_tiles * n_seqs * nkv;
        if ((g_wide == 2 || (g_wide == 1 && wide_blocks >= WIDE_MIN_BLOCKS)) && wide_blocks <= 0x7fffffffll) {
            p.n_row_tiles = (int)wide_tiles;
            return launch_wide((unsigned)wide_blocks, map_q, map_k, map_v, p, st);
        }
        p.n_row_tiles = (max_new + tpb - 1) / tpb;
        const long long blocks = (long long)p.n_row_tiles * n_seqs * nkv;
        if (blocks > 0x7fffffffll) return UB_ERR_ARG;
        return launch_attn<2, false>(dim3((unsigned)blocks), map_q, map_k, map_v, p, st);
    }
    if (max_new != 1) return UB_ERR_ARG;
    if (p.n_slices > 1 && (!part_o || !part_ml || ((uintptr_t)part_o & 15))) return UB_ERR_ARG;
    int rc = launch_attn<DECODE_STAGES, true>(dim3(p.n_slices, n_seqs, nkv), map_q, map_k, map_v, p, st);
    if (rc != 0 || p.n_slices == 1) return rc;
    cudaError_t e = ub_launch_dependent(attn_tc_combine_kernel, dim3(n_seqs * nh), dim3(HD), 0, st, p);
    return (int)e;
}
