// Attention over the paged bfloat16 cache on the tensor cores, for one head size fixed at
// compile time (-DHEAD_DIM=..., any multiple of 16 up to 256).
//
// Two kernels share the inner tile code (flash attention: scores, running maximum and sum in
// float32, probabilities rounded to bfloat16 for the second product):
//   prefill  one CTA for 64 rows of one KV head, a row being (token, query head of the group);
//            the group's heads share every K/V tile that is loaded.  4 warps x 16 rows.
//   decode   one new token a sequence: one CTA for (slice of the keys, sequence, KV head); its
//            4 warps take every fourth 16 keys of each 64-key tile and their partial results
//            are merged in shared memory; with several slices the CTA writes an unnormalised
//            partial result (maximum, sum, output) that attn_combine merges.
// K and V tiles are one cache page (64 positions of one KV head, contiguous) and arrive with
// cp.async, double buffered.  Positions the sequence has not reached are written as zeros into
// shared memory, so whatever the cache held before cannot reach the result.
//
// The arithmetic restated is the reference's per-token loop (src/model/qwen_block.cpp:94-135):
// scores q.k * scale over the visible positions (p - window, p], max-shifted softmax, weighted
// sum of values, query head h on KV head h / (heads / kv heads).
#include "attn_device.cuh"

struct AttnParams {
    const bf16* q; long long q_stride;
    bf16* out; long long o_stride;
    const bf16* kc; const bf16* vc;
    const int* seq_start; const int* seq_before;
    int nh, group, window;
    float c;                                  // scale * log2(e)
    float* part_o; float* part_ml;            // decode with several slices
    int n_slices;
};

// ---------------------------------------------------------------------------------------
// prefill: grid (row tiles of the longest sequence, sequences, KV heads)
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(NTHREADS)
attn_prefill_kernel(AttnParams p, PagedKV c) {
    extern __shared__ __align__(16) uint8_t smem_raw[];
    pdl_trigger();
    pdl_wait();
    bf16* Qs = (bf16*)smem_raw;                    // [64][LDS]
    bf16* Ks = Qs + 64 * LDS;                      // [2][64][LDS]
    bf16* Vs = Ks + 2 * KT * LDS;                  // [2][64][LDS]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int seq = blockIdx.y, kvh = blockIdx.z;
    const int q0 = p.seq_start[seq], q_len = p.seq_start[seq + 1] - q0, before = p.seq_before[seq];
    const int G = p.group;
    const int R0 = blockIdx.x * 64;                // first row of this tile; row = token * G + head in group
    if (R0 >= q_len * G) return;
    const int last_pos = before + q_len - 1;

    // Q rows of the tile into shared memory (rows past the sequence's end: zeros)
    constexpr int CH = HD / 8;
    for (int i = tid; i < 64 * CH; i += NTHREADS) {
        const int r = i / CH, ch = i % CH;
        const int R = R0 + r, tok = R / G, g = R % G;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (tok < q_len) v = *reinterpret_cast<const uint4*>(p.q + (long long)(q0 + tok) * p.q_stride + (long long)(kvh * G + g) * HD + ch * 8);
        *reinterpret_cast<uint4*>(Qs + r * LDS + ch * 8) = v;
    }
    // this thread's two rows
    int row_pos[2]; bool row_ok[2]; int row_tok[2], row_g[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int R = R0 + warp * 16 + (lane >> 2) + r * 8;
        row_tok[r] = R / G; row_g[r] = R % G;
        row_ok[r] = row_tok[r] < q_len;
        row_pos[r] = before + row_tok[r];
    }
    const int tok_first = R0 / G, tok_last = min(q_len - 1, (R0 + 63) / G);
    const int pos_hi = before + tok_last;
    int pos_lo = 0;
    if (p.window > 0) pos_lo = max(0, before + tok_first - p.window + 1);
    const int t_lo = pos_lo / KT, t_hi = pos_hi / KT;

    float o[DTILES][4];
#pragma unroll
    for (int dt = 0; dt < DTILES; ++dt) o[dt][0] = o[dt][1] = o[dt][2] = o[dt][3] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

    load_kv_tile(Ks, Vs, p.kc, p.vc, c, seq, kvh, t_lo * KT, last_pos, tid);
    cp_async_commit();
    for (int t = t_lo; t <= t_hi; ++t) {
        const int buf = (t - t_lo) & 1;
        if (t < t_hi) {
            load_kv_tile(Ks + (buf ^ 1) * KT * LDS, Vs + (buf ^ 1) * KT * LDS, p.kc, p.vc, c, seq, kvh, (t + 1) * KT, last_pos, tid);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const bf16* K = Ks + buf * KT * LDS;
        const bf16* V = Vs + buf * KT * LDS;
        float s[8][4];
        scores<8>(s, Qs, warp * 16, K, 0, lane);
        softmax_step<8>(s, o, m, l, p.c, row_pos, row_ok, t * KT, p.window, lane);
        weighted_values<8>(o, s, V, 0, lane);
        __syncthreads();                             // the buffer is loaded again two tiles on
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        if (!row_ok[r]) continue;
        const float inv = 1.0f / l[r];
        bf16* dst = p.out + (long long)(q0 + row_tok[r]) * p.o_stride + (long long)(kvh * G + row_g[r]) * HD + (lane & 3) * 2;
#pragma unroll
        for (int dt = 0; dt < DTILES; ++dt)
            *reinterpret_cast<uint32_t*>(dst + dt * 8) = pack_bf16(o[dt][2 * r] * inv, o[dt][2 * r + 1] * inv);
    }
}

// ---------------------------------------------------------------------------------------
// decode: one new token a sequence; grid (slices, sequences, KV heads); group <= 16
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(NTHREADS)
attn_decode_kernel(AttnParams p, PagedKV c) {
    extern __shared__ __align__(16) uint8_t smem_raw[];
    pdl_trigger();
    pdl_wait();
    bf16* Qs = (bf16*)smem_raw;                    // [16][LDS]
    bf16* Ks = Qs + 16 * LDS;                      // [DSTAGES][64][LDS]
    bf16* Vs = Ks + DSTAGES * KT * LDS;
    float* red = ATTN_ALIAS ? (float*)Ks : (float*)(Vs + DSTAGES * KT * LDS);   // [4 warps][16 rows][HD + 2]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int slice = blockIdx.x, seq = blockIdx.y, kvh = blockIdx.z;
    const int G = p.group;
    const int row = p.seq_start[seq];              // the sequence's one token
    const int pos = p.seq_before[seq];             // its position; keys [lo, pos]
    int lo = 0;
    if (p.window > 0) lo = max(0, pos - p.window + 1);
    const int t_first = lo / KT, t_last = pos / KT;
    const int n_tiles = t_last - t_first + 1;
    const int per = (n_tiles + p.n_slices - 1) / p.n_slices;
    const int t_lo = t_first + slice * per, t_hi = min(t_last, t_lo + per - 1);

    constexpr int CH = HD / 8;
    for (int i = tid; i < 16 * CH; i += NTHREADS) {
        const int r = i / CH, ch = i % CH;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (r < G) v = *reinterpret_cast<const uint4*>(p.q + (long long)row * p.q_stride + (long long)(kvh * G + r) * HD + ch * 8);
        *reinterpret_cast<uint4*>(Qs + r * LDS + ch * 8) = v;
    }
    int row_pos[2] = {pos, pos};
    bool row_ok[2] = {(lane >> 2) < G, (lane >> 2) + 8 < G};
    float o[DTILES][4];
#pragma unroll
    for (int dt = 0; dt < DTILES; ++dt) o[dt][0] = o[dt][1] = o[dt][2] = o[dt][3] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

    // a ring of DSTAGES tiles: DSTAGES - 1 tiles are on their way while one is used.  One group of
    // copies is committed for every tile slot, empty past the end, so the count to wait for is fixed.
#pragma unroll
    for (int i = 0; i < DSTAGES - 1; ++i) {
        if (t_lo + i <= t_hi)
            load_kv_tile(Ks + i * KT * LDS, Vs + i * KT * LDS, p.kc, p.vc, c, seq, kvh, (t_lo + i) * KT, pos, tid);
        cp_async_commit();
    }
    for (int t = t_lo; t <= t_hi; ++t) {
        const int buf = (t - t_lo) % DSTAGES;
        const int ahead = t + DSTAGES - 1;
        if (ahead <= t_hi) {
            const int nb = (ahead - t_lo) % DSTAGES;
            load_kv_tile(Ks + nb * KT * LDS, Vs + nb * KT * LDS, p.kc, p.vc, c, seq, kvh, ahead * KT, pos, tid);
        }
        cp_async_commit();
        cp_async_wait<DSTAGES - 1>();
        __syncthreads();
        float s[2][4];
        scores<2>(s, Qs, 0, Ks + buf * KT * LDS, warp * 16, lane);
        softmax_step<2>(s, o, m, l, p.c, row_pos, row_ok, t * KT + warp * 16, p.window, lane);
        weighted_values<2>(o, s, Vs + buf * KT * LDS, warp * 16, lane);
        __syncthreads();                             // the slot is filled again at the next step
    }
    cp_async_wait<0>();
    __syncthreads();                                 // K/V no longer needed: the merge buffer lies over them
    // merge the four warps: each has (m, l, o) over its keys
    constexpr int RS = HD + 2;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        float* dst = red + ((warp * 16) + (lane >> 2) + r * 8) * RS;
#pragma unroll
        for (int dt = 0; dt < DTILES; ++dt) {
            dst[dt * 8 + (lane & 3) * 2] = o[dt][2 * r];
            dst[dt * 8 + (lane & 3) * 2 + 1] = o[dt][2 * r + 1];
        }
        if ((lane & 3) == 0) { dst[HD] = m[r]; dst[HD + 1] = l[r]; }
    }
    __syncthreads();
    for (int i = tid; i < G * HD; i += NTHREADS) {
        const int g = i / HD, d = i % HD;
        float mm = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) mm = fmaxf(mm, red[(w * 16 + g) * RS + HD]);
        float acc = 0.f, ll = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float mw = red[(w * 16 + g) * RS + HD];
            const float f = mw == -INFINITY ? 0.f : exp2f(mw - mm);
            acc += f * red[(w * 16 + g) * RS + d];
            ll += f * red[(w * 16 + g) * RS + HD + 1];
        }
        const int head = kvh * G + g;
        if (p.n_slices == 1) {
            p.out[(long long)row * p.o_stride + (long long)head * HD + d] = __float2bfloat16_rn(acc / ll);
        } else {
            const long long pi = ((long long)seq * p.nh + head) * p.n_slices + slice;
            p.part_o[pi * HD + d] = acc;
            if (d == 0) { p.part_ml[pi * 2] = mm; p.part_ml[pi * 2 + 1] = ll; }
        }
    }
}

// merge the slices of a decode step: grid (sequences * heads), HD threads (rounded up to a warp)
__global__ void attn_combine_kernel(AttnParams p) {
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
        if (d < HD) acc += f * p.part_o[(base + s) * HD + d];
    }
    if (d < HD) p.out[(long long)p.seq_start[seq] * p.o_stride + (long long)head * HD + d] = __float2bfloat16_rn(acc / ll);
}

// ---------------------------------------------------------------------------------------
UB_API int ub_attn_head_dim() { return HD; }

// mode 0: prefill kernel (any numbers of new tokens), mode 1: decode kernel (one new token for
// every sequence, group <= 16).  part_o: float32 [n_seqs, nh, n_slices, HD], part_ml: [.., 2].
UB_API int ub_attn_mma(int mode, const void* q, long long q_stride, void* out, long long o_stride, const void* kcache,
                       const void* vcache, const int* seq_start, const int* seq_before, const int* table,
                       int pages_per_seq, int ring, int page, int n_seqs, int max_new, int nh, int nkv, int window,
                       float scale, int n_slices, float* part_o, float* part_ml, cudaStream_t st) {
    if (n_seqs <= 0) return 0;
    if (page != KT || ring % page != 0 || nh % nkv != 0 || (q_stride % 8) != 0 || (o_stride % 2) != 0) return UB_ERR_ARG;
    if (((uintptr_t)q & 15) || ((uintptr_t)out & 3) || ((uintptr_t)kcache & 15) || ((uintptr_t)vcache & 15)) return UB_ERR_ARG;
    if (n_seqs > 65535 || nkv > 65535) return UB_ERR_ARG;
    PagedKV c{table, pages_per_seq, ring, page, nkv, HD};
    AttnParams p;
    p.q = (const bf16*)q; p.q_stride = q_stride; p.out = (bf16*)out; p.o_stride = o_stride;
    p.kc = (const bf16*)kcache; p.vc = (const bf16*)vcache; p.seq_start = seq_start; p.seq_before = seq_before;
    p.nh = nh; p.group = nh / nkv; p.window = window; p.c = scale * 1.4426950408889634f;
    p.part_o = part_o; p.part_ml = part_ml; p.n_slices = n_slices < 1 ? 1 : n_slices;
    static bool attr_done = false;
    const size_t sm_pre = (size_t)(64 + 4 * KT) * LDS * sizeof(bf16);
    const size_t sm_kv = (size_t)2 * DSTAGES * KT * LDS * sizeof(bf16), sm_red = (size_t)64 * (HD + 2) * sizeof(float);
    const size_t sm_dec = (size_t)16 * LDS * sizeof(bf16) + (ATTN_ALIAS ? (sm_kv > sm_red ? sm_kv : sm_red) : sm_kv + sm_red);
    if (!attr_done) {
        cudaError_t e = cudaFuncSetAttribute(attn_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm_pre);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(attn_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm_dec);
        if (e != cudaSuccess) return (int)e;
        attr_done = true;
    }
    if (mode == 0) {
        const int tiles = (max_new * p.group + 63) / 64;
        if (tiles < 1) return 0;
        dim3 grid(tiles, n_seqs, nkv);
        cudaError_t e = ub_launch_dependent(attn_prefill_kernel, grid, dim3(NTHREADS), sm_pre, st, p, c);
        if (e != cudaSuccess) return (int)e;
    } else {
        if (p.group > 16 || max_new != 1) return UB_ERR_ARG;
        if (p.n_slices > 1 && (!part_o || !part_ml)) return UB_ERR_ARG;
        dim3 grid(p.n_slices, n_seqs, nkv);
        cudaError_t e = ub_launch_dependent(attn_decode_kernel, grid, dim3(NTHREADS), sm_dec, st, p, c);
        if (e != cudaSuccess) return (int)e;
        if (p.n_slices > 1) {
            e = ub_launch_dependent(attn_combine_kernel, dim3(n_seqs * nh), dim3(((HD + 31) / 32) * 32), 0, st, p);
            if (e != cudaSuccess) return (int)e;
        }
    }
    UB_LAUNCH_CHECK();
    return 0;
}


// ---------------------------------------------------------------------------------------
// decode with TMA: the same arithmetic as attn_decode_kernel, for head sizes that are multiples
// of 64.  A fifth warp issues one TMA copy for each 64-column block of a K or V page (128-byte
// swizzle) into a ring of TSTAGES tiles guarded by mbarriers; the four computing warps never meet
// at a CTA-wide barrier inside the loop: each waits for a tile, uses its own 16 keys of it and
// gives the slot back.  ldmatrix addresses undo the swizzle (16-byte piece c of row r lies at
// piece c ^ (r % 8)), which also makes them free of bank conflicts.
// ---------------------------------------------------------------------------------------
#if HEAD_DIM % 64 == 0

struct TmaDecodeParams {
    AttnParams a;
    const int* table; int pages_per_seq, ring, nkv;
    int* error;
    FusedQKV f;
};

__global__ void __launch_bounds__(TMA_THREADS)
attn_decode_tma_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, TmaDecodeParams tp) {
    extern __shared__ uint8_t smem_raw[];
    pdl_trigger();
    const AttnParams& p = tp.a;
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* ring = smem;                                  // [TSTAGES][K page | V page]
    float* red = (float*)smem;                             // the merge buffer lies over the ring, after the loop
    bf16* Qs = (bf16*)(smem + TSTAGES * 2 * PAGE_BYTES);   // [16][LDS]
    uint64_t* full = (uint64_t*)(Qs + 16 * LDS);
    uint64_t* empty = full + TSTAGES;
    volatile int* err = (volatile int*)(empty + TSTAGES);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int slice = blockIdx.x, seq = blockIdx.y, kvh = blockIdx.z;
    const int G = p.group;
    const int row = p.seq_start[seq];
    const int pos = p.seq_before[seq];
    int lo = 0;
    if (p.window > 0) lo = max(0, pos - p.window + 1);
    const int t_first = lo / KT, t_last = pos / KT;
    const int all_tiles = t_last - t_first + 1;
    const int per = (all_tiles + p.n_slices - 1) / p.n_slices;
    const int t_lo = t_first + slice * per, t_hi = min(t_last, t_lo + per - 1);
    const int n_tiles = max(0, t_hi - t_lo + 1);

    if (tid == 0) {
        for (int s = 0; s < TSTAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 4); }
        *err = 0;
        fence_barrier_init();
    }
    __syncthreads();
    // One page of keys and values into stage j % TSTAGES of the ring.
    auto load_tile = [&](int j) {
        const int s = j % TSTAGES;
        const int posn = (t_lo + j) * KT;
        const int page = tp.table[(long long)seq * tp.pages_per_seq + (posn % tp.ring) / KT];
        const int r0 = (page * tp.nkv + kvh) * KT;
        uint8_t* st = ring + s * 2 * PAGE_BYTES;
        mbar_expect_tx(&full[s], 2 * PAGE_BYTES);
#pragma unroll
        for (int nb = 0; nb < NBLK; ++nb) {
            tma_load_2d(st + nb * BLK_BYTES, &map_k, &full[s], nb * 64, r0);
            tma_load_2d(st + PAGE_BYTES + nb * BLK_BYTES, &map_v, &full[s], nb * 64, r0);
        }
    };
    // The pages before the one that takes this step's key and value were written by earlier steps:
    // their copies start while the kernel that prepares q and writes the new key still runs.
    int early = 0;
    if (warp == 4 && lane == 0) {
        prefetch_tmap(&map_k); prefetch_tmap(&map_v);
        while (early < n_tiles && early < TSTAGES && t_lo + early < t_last) { load_tile(early); ++early; }
    }
    // the new key and value, held by the warp that reads their row of the page (fused mode only)
    const FusedQKV& f = tp.f;
    const bool fused = FUSABLE && f.qkv != nullptr;
    const bool has_new = fused && f.kcache != nullptr && n_tiles > 0 && t_hi == t_last;
    const int new_row = pos % KT;
    float new_k[FE], new_v[FE];
    float co[FE], si[FE], gq[FE], gk[FE];
    if (fused && warp < 4) {
        // the tables and the norm weights are written by no kernel: fetched before the wait
        if (f.cs) {
            const int j0 = (lane & 15) * FE;
            load_vec<float, FE>(f.cs + (long long)pos * (HD / 2) + j0, co);
            load_vec<float, FE>(f.sn + (long long)pos * (HD / 2) + j0, si);
        }
        if (f.qw) load_vec<float, FE>(f.qw + lane * FE, gq);
        if (f.kw) load_vec<float, FE>(f.kw + lane * FE, gk);
    }
    pdl_wait();
    if (fused) {
        if (warp < 4) {
            const int heads_all = p.nh + 2 * tp.nkv;
            const float* trow = f.qkv + (long long)row * heads_all * HD;
            const bool mine = has_new && warp == new_row / 16;
            // this warp's first query head, and the new key and value if they are this warp's: one round of loads
            float first[3][FE];
            {
                const float* src[3] = {trow + (long long)(kvh * G + min(warp, G - 1)) * HD,
                                       trow + (long long)(p.nh + kvh) * HD, trow + (long long)(p.nh + tp.nkv + kvh) * HD};
                if (mine) fused_sums<3>(f, src, lane, first);
                else fused_sums<1>(f, src, lane, first);
            }
            for (int r = warp; r < 16; r += 4) {
                float v[FE];
                if (r < G) {
                    if (r == warp) {
#pragma unroll
                        for (int i = 0; i < FE; ++i) v[i] = first[0][i];
                    } else {
                        const float* src[1] = {trow + (long long)(kvh * G + r) * HD};
                        fused_sums<1>(f, src, lane, &v);
                    }
                    fused_finish(f, f.qw ? gq : nullptr, f.cs != nullptr, co, si, lane, v);
                } else {
#pragma unroll
                    for (int i = 0; i < FE; ++i) v[i] = 0.f;
                }
                store_vec<bf16, FE>(Qs + r * LDS + lane * FE, v);
            }
            if (mine) {
#pragma unroll
                for (int i = 0; i < FE; ++i) { new_k[i] = first[1][i]; new_v[i] = first[2][i]; }
                fused_finish(f, f.kw ? gk : nullptr, f.cs != nullptr, co, si, lane, new_k);
                const PagedKV c{tp.table, tp.pages_per_seq, tp.ring, KT, tp.nkv, HD};
                const long long at = paged_offset(c, seq, pos, kvh) + lane * FE;
                store_vec<bf16, FE>(f.kcache + at, new_k);
                store_vec<bf16, FE>(f.vcache + at, new_v);
            }
        }
    } else {
        constexpr int CH = HD / 8;
        for (int i = tid; i < 16 * CH; i += TMA_THREADS) {
            const int r = i / CH, ch = i % CH;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (r < G) v = *reinterpret_cast<const uint4*>(p.q + (long long)row * p.q_stride + (long long)(kvh * G + r) * HD + ch * 8);
            *reinterpret_cast<uint4*>(Qs + r * LDS + ch * 8) = v;
        }
    }
    __syncthreads();

    float o[DTILES][4];
#pragma unroll
    for (int dt = 0; dt < DTILES; ++dt) o[dt][0] = o[dt][1] = o[dt][2] = o[dt][3] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

    if (warp == 4) {
        if (lane == 0) {
            int armed = early;
            for (int j = early; j < n_tiles; ++j) {
                const int s = j % TSTAGES;
                if (!mbar_wait(&empty[s], (uint32_t)(((j / TSTAGES) & 1) ^ 1), err)) break;
                load_tile(j);
                armed = j + 1;
            }
            if (*err) {
                const long long tstart = clock64();
                for (int j = max(0, armed - TSTAGES); j < armed; ++j)
                    while (!mbar_try_wait(&full[j % TSTAGES], (j / TSTAGES) & 1)) if (clock64() - tstart > WAIT_LIMIT_CYCLES / 4) break;
            }
        }
    } else {
        int row_pos[2] = {pos, pos};
        bool row_ok[2] = {(lane >> 2) < G, (lane >> 2) + 8 < G};
        for (int j = 0; j < n_tiles; ++j) {
            const int s = j % TSTAGES;
            if (!mbar_wait(&full[s], (uint32_t)((j / TSTAGES) & 1), err)) break;
            const uint32_t k_base = smem_u32(ring + s * 2 * PAGE_BYTES), v_base = k_base + PAGE_BYTES;
            const int base = (t_lo + j) * KT;
            if (has_new && t_lo + j == t_last && warp == new_row / 16) {
                // the page came from the cache as it was before this step: the new key and value go in here
                uint8_t* pg = ring + s * 2 * PAGE_BYTES;
                store_vec<bf16, FE>(reinterpret_cast<bf16*>(pg + swz(new_row, lane * FE)), new_k);
                store_vec<bf16, FE>(reinterpret_cast<bf16*>(pg + PAGE_BYTES + swz(new_row, lane * FE)), new_v);
                __syncwarp();
            }
            if (base + KT - 1 > pos) {
                // this warp's rows of V past the sequence's end: zeros instead of what the page held before
                for (int i = lane; i < 16 * NBLK * 8; i += 32) {
                    const int r = warp * 16 + i / (NBLK * 8), rest = i % (NBLK * 8);
                    if (base + r > pos)
                        *reinterpret_cast<uint4*>(ring + s * 2 * PAGE_BYTES + PAGE_BYTES + (rest / 8) * BLK_BYTES + r * 128 + (rest % 8) * 16) = make_uint4(0, 0, 0, 0);
                }
                __syncwarp();
            }
            float sc[2][4];
            scores_swz<2>(sc, Qs, k_base, warp * 16, lane);
            softmax_step<2>(sc, o, m, l, p.c, row_pos, row_ok, base + warp * 16, p.window, lane);
            weighted_values_swz<2>(o, sc, v_base, warp * 16, lane);
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[s]);
        }
    }
    __syncthreads();                                       // every tile is used: the ring becomes the merge buffer
    constexpr int RS = HD + 2;
    if (warp < 4) {
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            float* dst = red + ((warp * 16) + (lane >> 2) + r * 8) * RS;
#pragma unroll
            for (int dt = 0; dt < DTILES; ++dt) {
                dst[dt * 8 + (lane & 3) * 2] = o[dt][2 * r];
                dst[dt * 8 + (lane & 3) * 2 + 1] = o[dt][2 * r + 1];
            }
            if ((lane & 3) == 0) { dst[HD] = m[r]; dst[HD + 1] = l[r]; }
        }
    }
    __syncthreads();
    for (int i = tid; i < G * HD; i += TMA_THREADS) {
        const int g = i / HD, d = i % HD;
        float mm = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) mm = fmaxf(mm, red[(w * 16 + g) * RS + HD]);
        float acc = 0.f, ll = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float mw = red[(w * 16 + g) * RS + HD];
            const float f = mw == -INFINITY ? 0.f : exp2f(mw - mm);
            acc += f * red[(w * 16 + g) * RS + d];
            ll += f * red[(w * 16 + g) * RS + HD + 1];
        }
        const int head = kvh * G + g;
        if (p.n_slices == 1) {
            p.out[(long long)row * p.o_stride + (long long)head * HD + d] = __float2bfloat16_rn(acc / ll);
        } else {
            const long long pi = ((long long)seq * p.nh + head) * p.n_slices + slice;
            p.part_o[pi * HD + d] = acc;
            if (d == 0) { p.part_ml[pi * 2] = mm; p.part_ml[pi * 2 + 1] = ll; }
        }
    }
    if (tid == 0 && *err) atomicExch(tp.error, 1);
}

// tensor map of one run's K or V cache [pages, kv heads, 64, HD] as rows of HD, boxes of 64 columns x 64 rows
UB_API int ub_attn_map_kv(void* out_map, const void* cache, long long n_pages, int nkv) {
    EncodeTiledFn enc = tensor_map_encoder();
    if (!enc) return UB_ERR_UNSUPPORTED;
    if (((uintptr_t)cache & 15) || n_pages < 1) return UB_ERR_ARG;
    cuuint64_t dims[2] = {(cuuint64_t)HD, (cuuint64_t)(n_pages * nkv * KT)};
    cuuint64_t strides[1] = {(cuuint64_t)HD * 2};
    cuuint32_t box[2] = {64, (cuuint32_t)KT};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc((CUtensorMap*)out_map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (void*)cache, dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : UB_ERR_ARG;
}

UB_API int ub_attn_decode_tma_stages() { return TSTAGES; }

// one new token for every sequence, group <= 16; K and V through their tensor maps
static int decode_tma_launch(const void* map_k, const void* map_v, const void* q, long long q_stride, void* out,
                             long long o_stride, const int* seq_start, const int* seq_before, const int* table,
                             int pages_per_seq, int ring, int page, int n_seqs, int nh, int nkv, int window,
                             float scale, int n_slices, float* part_o, float* part_ml, int* error, const FusedQKV& f,
                             cudaStream_t st) {
    if (n_seqs <= 0) return 0;
    if (page != KT || ring % page != 0 || nh % nkv != 0 || (q_stride % 8) != 0 || (o_stride % 2) != 0) return UB_ERR_ARG;
    if (((uintptr_t)q & 15) || ((uintptr_t)out & 3) || n_seqs > 65535 || nkv > 65535 || nh / nkv > 16) return UB_ERR_ARG;
    TmaDecodeParams tp;
    tp.f = f;
    AttnParams& p = tp.a;
    p.q = (const bf16*)q; p.q_stride = q_stride; p.out = (bf16*)out; p.o_stride = o_stride;
    p.kc = nullptr; p.vc = nullptr; p.seq_start = seq_start; p.seq_before = seq_before;
    p.nh = nh; p.group = nh / nkv; p.window = window; p.c = scale * 1.4426950408889634f;
    p.part_o = part_o; p.part_ml = part_ml; p.n_slices = n_slices < 1 ? 1 : n_slices;
    tp.table = table; tp.pages_per_seq = pages_per_seq; tp.ring = ring; tp.nkv = nkv; tp.error = error;
    if (p.n_slices > 1 && (!part_o || !part_ml)) return UB_ERR_ARG;
    const size_t sm_ring = (size_t)TSTAGES * 2 * PAGE_BYTES, sm_red = (size_t)64 * (HD + 2) * sizeof(float);
    const size_t sm = (sm_ring > sm_red ? sm_ring : sm_red) + (size_t)16 * LDS * sizeof(bf16) + 2 * TSTAGES * 8 + 16 + 1024;
    static bool attr_done = false;
    if (!attr_done) {
        cudaError_t e = cudaFuncSetAttribute(attn_decode_tma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);
        if (e != cudaSuccess) return (int)e;
        attr_done = true;
    }
    cudaError_t e = ub_launch_dependent(attn_decode_tma_kernel, dim3(p.n_slices, n_seqs, nkv), dim3(TMA_THREADS), sm, st,
                                        *(const CUtensorMap*)map_k, *(const CUtensorMap*)map_v, tp);
    if (e != cudaSuccess) return (int)e;
    if (p.n_slices > 1) {
        e = ub_launch_dependent(attn_combine_kernel, dim3(n_seqs * nh), dim3(((HD + 31) / 32) * 32), 0, st, p);
        if (e != cudaSuccess) return (int)e;
    }
    return 0;
}

UB_API int ub_attn_decode_tma(const void* map_k, const void* map_v, const void* q, long long q_stride, void* out,
                              long long o_stride, const int* seq_start, const int* seq_before, const int* table,
                              int pages_per_seq, int ring, int page, int n_seqs, int nh, int nkv, int window,
                              float scale, int n_slices, float* part_o, float* part_ml, int* error, cudaStream_t st) {
    FusedQKV f{};
    return decode_tma_launch(map_k, map_v, q, q_stride, out, o_stride, seq_start, seq_before, table, pages_per_seq,
                             ring, page, n_seqs, nh, nkv, window, scale, n_slices, part_o, part_ml, error, f, st);
}

// The same from the fused projection's result instead of q: qkv [n_parts][tokens, (nh + 2 nkv) * HD]
// float32, its parts part_stride elements apart and summed here; qw, kw [HD] norm weights (null: no
// norm); cs, sn [max_pos, HD / 2] (null: no rotation); kcache, vcache: where the new key and value
// are written (null: this layer reads a cache that another layer has written).  Head sizes 64, 128, 256.
UB_API int ub_attn_decode_tma_qkv(const void* map_k, const void* map_v, const float* qkv, int n_parts,
                                  long long part_stride, const float* qw, const float* kw, const float* cs,
                                  const float* sn, float eps, void* kcache, void* vcache, void* out, long long o_stride,
                                  const int* seq_start, const int* seq_before, const int* table, int pages_per_seq,
                                  int ring, int page, int n_seqs, int nh, int nkv, int window, float scale,
                                  int n_slices, float* part_o, float* part_ml, int* error, cudaStream_t st) {
    if (!FUSABLE) return UB_ERR_UNSUPPORTED;
    if (!qkv || n_parts < 1 || (part_stride % 4) != 0 || (!kcache) != (!vcache) || (!cs) != (!sn)) return UB_ERR_ARG;
    if ((((uintptr_t)qkv | (uintptr_t)qw | (uintptr_t)kw | (uintptr_t)cs | (uintptr_t)sn | (uintptr_t)kcache |
          (uintptr_t)vcache) & 15) != 0) return UB_ERR_ARG;
    FusedQKV f{qkv, n_parts, part_stride, qw, kw, cs, sn, eps, (bf16*)kcache, (bf16*)vcache};
    return decode_tma_launch(map_k, map_v, nullptr, 0, out, o_stride, seq_start, seq_before, table, pages_per_seq,
                             ring, page, n_seqs, nh, nkv, window, scale, n_slices, part_o, part_ml, error, f, st);
}
#endif   // HEAD_DIM % 64 == 0

// ---------------------------------------------------------------------------------------
// decode attention without any allocation: see attn_noalloc.h
// ---------------------------------------------------------------------------------------
#include "attn_noalloc.h"

// Partial results of the key slices: [o floats | (max, sum) floats].  Part of the library's
// device image; in host code this name is only a handle, never a device address.
static __device__ __align__(256) float g_noalloc_scratch[UB_NOALLOC_SCRATCH_O_FLOATS + UB_NOALLOC_SCRATCH_ML_FLOATS];

constexpr int NOALLOC_MAX_DEVICES = 64;
static float* g_noalloc_ptr[NOALLOC_MAX_DEVICES] = {};

UB_API int ub_attn_decode_noalloc(const void* q, long long q_stride, void* out, long long o_stride, const void* kcache,
                                  const void* vcache, const int* seq_start, const int* seq_before, const int* table,
                                  int pages_per_seq, int ring, int page, int n_seqs, int nh, int nkv, int window,
                                  float scale, int n_slices, cudaStream_t st) {
    if (n_seqs <= 0) return 0;
    if (n_slices < 1 || nh < 1) return UB_ERR_ARG;
    const long long parts = (long long)n_seqs * nh * n_slices;
    if (parts * HD > UB_NOALLOC_SCRATCH_O_FLOATS || parts * 2 > UB_NOALLOC_SCRATCH_ML_FLOATS) return UB_ERR_NOALLOC_TOO_LARGE;
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= NOALLOC_MAX_DEVICES) return UB_ERR_ARG;
    if (!g_noalloc_ptr[dev]) {
        // set-up, once a device, with that device current: the array's address on this device
        float* ptr = nullptr;
        e = cudaGetSymbolAddress((void**)&ptr, g_noalloc_scratch);
        if (e != cudaSuccess) return (int)e;
        if (!ptr) return UB_ERR_ARG;
        g_noalloc_ptr[dev] = ptr;
    }
    float* part_o = g_noalloc_ptr[dev];
    float* part_ml = part_o + UB_NOALLOC_SCRATCH_O_FLOATS;
    return ub_attn_mma(1, q, q_stride, out, o_stride, kcache, vcache, seq_start, seq_before, table, pages_per_seq, ring,
                       page, n_seqs, 1, nh, nkv, window, scale, n_slices, part_o, part_ml, st);
}
