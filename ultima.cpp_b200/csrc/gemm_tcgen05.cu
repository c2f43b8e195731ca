// Matrix product on the fifth-generation tensor cores: out[t, n] = sum_k A[t, k] * W[n, k],
// bfloat16 operands, float32 accumulation in tensor memory.
//
// The weight matrix is the M operand of the MMA (128 rows of W a tile) and the tokens are the
// N operand (16 to 256 tokens a tile).  A prompt of thousands of tokens and a decode step of one
// token are the same kernel with another token tile: with few tokens the kernel streams the
// weights once at memory speed, with many it is bound by the tensor cores.  Both operands are
// K-major, which is how activations [tokens, k] and weights [out, k] lie in memory.
//
// One CTA computes one tile (optionally one slice of K).  Warp 0 issues the TMA loads (weights
// and activations, 64 k-columns = 128 bytes a row, 128-byte swizzle) into a ring of stages;
// warp 1 allocates tensor memory and issues tcgen05.mma from one thread; warps 2-5 read the
// accumulators back with tcgen05.ld (each warp its quarter of the 128 lanes = weight rows) and
// apply the epilogue: store (bfloat16 or float32), add into a float32 matrix (the residual
// stream; with atomics when K is split), or silu(gate) * up from two accumulators fed by two
// weight tiles.  Every wait on an mbarrier has a time limit; on a timeout the kernel raises a
// flag in global memory, lets its copies land, frees its tensor memory and returns.
//
// The reference computes these products with AVX2 row-dot kernels in float32
// (src/kernels/dot_batched.cpp:39-96, src/model/weight_dispatch.cpp:374-441); the float32
// restatement of that is gemm_simt.cu, which this kernel is tested against.
#include "common.cuh"
#include "tc_common.cuh"

// EPI_SWIGLU: two weight tiles (gate rows, up rows) and two accumulators.  EPI_SWIGLU_IL: one weight
// matrix in which blocks of 64 gate rows and 64 up rows alternate, one accumulator whose lanes
// 0-63 are gate and 64-127 up of the same 64 features; the halves meet through shared memory.
enum : int { EPI_STORE = 0, EPI_ADD = 1, EPI_SWIGLU = 2, EPI_SWIGLU_IL = 3 };

constexpr int BM = 128;              // weight rows a tile (MMA M)
constexpr int BK = 64;               // k columns a stage: 128 bytes of bfloat16
constexpr int UMMA_K = 16;
constexpr int NUM_THREADS = 192;

// Instruction descriptor: float32 accumulate, bfloat16 A and B, both K-major, M = 128, N = n.
__host__ __device__ constexpr uint32_t make_idesc(int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}

struct GemmParams {
    void* out;            // [T, N] (element type by the kernel's template)
    long long ldo;        // row stride of out, elements
    long long split_stride;   // elements between the partial results of K slices (EPI_STORE float32), else 0
    int T, N, K;
    int kb_per_split;     // 64-column blocks of K a slice
    int atomic;           // EPI_ADD: add with atomics (K is split)
    int share_tail;       // persistent EPI_ADD: the tiles of the last, part-empty round are shared out by k blocks
    int* error;           // raised on a timeout
};

template <int BN, int EPI>
struct Smem {
    static constexpr int A_BYTES = BM * BK * 2;
    static constexpr int B_BYTES = BN * BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES * (EPI == EPI_SWIGLU ? 2 : 1) + B_BYTES;
    // token tiles of up to 64 leave room for two CTAs on an SM (this kernel's and the next one's)
    static constexpr int BUDGET = (BN <= 64 && EPI != EPI_SWIGLU ? 110 : 196) * 1024;
    static constexpr int STAGES_RAW = BUDGET / STAGE_BYTES;
    static constexpr int STAGES = STAGES_RAW > 10 ? 10 : STAGES_RAW;
    // (the interleaved gate product's exchange buffer, 4 KB, lies over the first stage: the epilogue runs when
    // every stage has been used for the last time)
    static constexpr int TOTAL = STAGES * STAGE_BYTES + 1024 /*alignment*/ + 256 /*barriers*/;
    static_assert(STAGE_BYTES >= 64 * 16 * 4, "the exchange buffer must fit a stage");
    static constexpr int ACC_COLS = BN * (EPI == EPI_SWIGLU ? 2 : 1);
    static constexpr int TMEM_COLS = ACC_COLS <= 32 ? 32 : ACC_COLS <= 64 ? 64 : ACC_COLS <= 128 ? 128 : ACC_COLS <= 256 ? 256 : 512;
};

// The epilogue of one tile: this thread's accumulator lane (weight row n0 + 32 q + lane), all token
// columns, in pieces of 16.  ``tile_w`` is the index of the 128-row weight tile, ``slice`` the K slice.
template <int BN, int EPI, typename TO>
__device__ __forceinline__ void epilogue_tile(const GemmParams& p, uint32_t tmem_acc, int q, int lane, int tile_w,
                                              int t0, int slice, float* xch) {
    const int n = tile_w * BM + q * 32 + lane;
    TO* out = (TO*)p.out + (EPI == EPI_STORE ? (long long)slice * p.split_stride : 0);
#pragma unroll 1
    for (int c0 = 0; c0 < BN; c0 += 16) {
        if (t0 + c0 >= p.T) break;               // uniform over the epilogue warps
        uint32_t r[16], r2[16];
        const uint32_t taddr = tmem_acc + ((uint32_t)(q * 32) << 16) + (uint32_t)c0;
        tmem_ld16(taddr, r);
        if (EPI == EPI_SWIGLU) tmem_ld16(taddr + BN, r2);
        tmem_ld_wait();
        if (EPI == EPI_SWIGLU_IL) {
            // lanes 64..127 hold "up" of the 64 features whose "gate" lanes 0..63 hold.  The halves
            // swap through shared memory: gate threads finish columns 0..7, up threads 8..15.
            const int fl = (q & 1) * 32 + lane;               // feature within the tile's 64
            const bool up = q >= 2;
#pragma unroll
            for (int c = 0; c < 8; ++c) xch[((up ? 0 : 8) + c) * 64 + fl] = __uint_as_float(up ? r[c] : r[8 + c]);
            asm volatile("bar.sync 1, 128;" ::: "memory");
            const int f = tile_w * 64 + fl;
            if (f < p.N / 2) {
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    const int col = (up ? 8 : 0) + c;
                    const int t = t0 + c0 + col;
                    if (t >= p.T) break;
                    const float own = __uint_as_float(up ? r[8 + c] : r[c]), other = xch[col * 64 + fl];
                    const float g = up ? other : own, u = up ? own : other;
                    out[(long long)t * p.ldo + f] = from_f32<TO>(g / (1.0f + __expf(-g)) * u);
                }
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
        } else if (n < p.N) {
#pragma unroll
            for (int c = 0; c < 16; ++c) {
                const int t = t0 + c0 + c;
                if (t >= p.T) break;
                const float v = __uint_as_float(r[c]);
                TO* dst = out + (long long)t * p.ldo + n;
                if (EPI == EPI_STORE) *dst = from_f32<TO>(v);
                else if (EPI == EPI_ADD) {
                    // a reduction at the memory side: no load, no wait; one writer an element
                    // unless K is split, so the sum's order is fixed in that case
                    asm volatile("red.global.add.f32 [%0], %1;" ::"l"(dst), "f"(v) : "memory");
                } else {
                    const float u = __uint_as_float(r2[c]);
                    *dst = from_f32<TO>(v / (1.0f + __expf(-v)) * u);
                }
            }
        }
    }
}

template <int BN, int EPI, typename TO>
__global__ void __launch_bounds__(NUM_THREADS)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_w2,
               const __grid_constant__ CUtensorMap map_a, GemmParams p) {
    using S = Smem<BN, EPI>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* full = (uint64_t*)(smem + S::STAGES * S::STAGE_BYTES);
    uint64_t* empty = full + S::STAGES;
    uint64_t* acc_full = empty + S::STAGES;
    uint32_t* tmem_slot = (uint32_t*)(acc_full + 1);
    volatile int* err = (volatile int*)(tmem_slot + 1);
    float* xch = (float*)smem;                   // EPI_SWIGLU_IL only: over the first stage, which is free by then

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * BM;                 // first weight row = first output column
    const int t0 = blockIdx.y * BN;                 // first token
    const int nkb_all = (p.K + BK - 1) / BK;
    const int kb0 = blockIdx.z * p.kb_per_split;
    const int kb1 = min(nkb_all, kb0 + p.kb_per_split);
    const int nkb = kb1 - kb0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < S::STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        mbar_init(acc_full, 1);
        *err = 0;
        fence_barrier_init();
    }
    if (warp == 1) { tmem_alloc(tmem_slot, S::TMEM_COLS); tmem_relinquish(); }
    if (warp == 0 && lane == 0) {
        prefetch_tmap(&map_w); prefetch_tmap(&map_a);
        if (EPI == EPI_SWIGLU) prefetch_tmap(&map_w2);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_trigger();                                       // the next kernel may begin its own prologue

    if (warp == 0) {
        // ---------------- producer ----------------
        // Weights do not depend on the kernel before this one: their loads start at once and fill
        // the ring while that kernel still runs.  Activations are loaded after it has ended.
        if (lane == 0) {
            int armed = 0;
            const int pre = min(nkb, S::STAGES);
            for (int i = 0; i < pre; ++i) {                 // fresh barriers: nothing to wait for
                uint8_t* st = smem + i * S::STAGE_BYTES;
                mbar_expect_tx(&full[i], S::STAGE_BYTES);
                const int kx = (kb0 + i) * BK;
                tma_load_2d(st, &map_w, &full[i], kx, n0);
                if (EPI == EPI_SWIGLU) tma_load_2d(st + S::A_BYTES, &map_w2, &full[i], kx, n0);
            }
            pdl_wait();
            for (int i = 0; i < pre; ++i) {
                uint8_t* st = smem + i * S::STAGE_BYTES;
                tma_load_2d(st + S::A_BYTES * (EPI == EPI_SWIGLU ? 2 : 1), &map_a, &full[i], (kb0 + i) * BK, t0);
                armed = i + 1;
            }
            for (int i = pre; i < nkb; ++i) {
                const int s = i % S::STAGES;
                const uint32_t ph = (i / S::STAGES) & 1;
                if (!mbar_wait(&empty[s], ph ^ 1, err)) break;
                uint8_t* st = smem + s * S::STAGE_BYTES;
                mbar_expect_tx(&full[s], S::STAGE_BYTES);
                const int kx = (kb0 + i) * BK;
                tma_load_2d(st, &map_w, &full[s], kx, n0);
                if (EPI == EPI_SWIGLU) tma_load_2d(st + S::A_BYTES, &map_w2, &full[s], kx, n0);
                tma_load_2d(st + S::A_BYTES * (EPI == EPI_SWIGLU ? 2 : 1), &map_a, &full[s], kx, t0);
                armed = i + 1;
            }
            if (*err) {
                // let the copies that are in flight land before the CTA's memory goes away
                for (int i = max(0, armed - S::STAGES); i < armed; ++i) {
                    const long long tstart = clock64();
                    while (!mbar_try_wait(&full[i % S::STAGES], (i / S::STAGES) & 1))
                        if (clock64() - tstart > WAIT_LIMIT_CYCLES / 8) break;
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc(BN);
            bool ok = true;
            for (int i = 0; i < nkb && ok; ++i) {
                const int s = i % S::STAGES;
                const uint32_t ph = (i / S::STAGES) & 1;
                ok = mbar_wait(&full[s], ph, err);
                if (!ok) break;
                tc_fence_after();
                const uint32_t a_addr = smem_u32(smem + s * S::STAGE_BYTES);
                const uint32_t b_addr = a_addr + S::A_BYTES * (EPI == EPI_SWIGLU ? 2 : 1);
                const uint64_t da = make_desc(a_addr), db = make_desc(b_addr);
                const uint64_t da2 = make_desc(a_addr + S::A_BYTES);
#pragma unroll
                for (int k = 0; k < BK / UMMA_K; ++k) {
                    const uint64_t koff = (uint64_t)((k * UMMA_K * 2) >> 4);       // 32 bytes a step
                    const uint32_t accum = (i > 0 || k > 0) ? 1u : 0u;
                    tc_mma_bf16(tmem_base, da + koff, db + koff, idesc, accum);
                    if (EPI == EPI_SWIGLU) tc_mma_bf16(tmem_base + BN, da2 + koff, db + koff, idesc, accum);
                }
                tc_commit(&empty[s]);            // the stage is free once these MMAs have read it
            }
            tc_commit(acc_full);                 // all MMAs done: accumulators complete
        }
    } else {
        // ---------------- epilogue: warps 2..5 ----------------
        const int q = warp & 3;                          // the lanes this warp may read: 32 q .. 32 q + 31
        pdl_wait();                                      // the output may be read by the kernel before
        bool ok = nkb > 0 ? mbar_wait(acc_full, 0, err) : true;
        tc_fence_after();
        if (ok && nkb > 0) epilogue_tile<BN, EPI, TO>(p, tmem_base, q, lane, blockIdx.x, t0, blockIdx.z, xch);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, S::TMEM_COLS);
    }
    if (threadIdx.x == 0 && *err) atomicExch(p.error, 1);
}

// ---------------------------------------------------------------------------------------
// The same product for many tiles a CTA: one CTA an SM walks over tiles c, c + G, c + 2G, ...
// The ring of stages never drains between tiles, and there are two accumulators in tensor
// memory, so the epilogue of one tile runs while the MMAs of the next are issued.
// ---------------------------------------------------------------------------------------
// The pieces of work of one CTA of the persistent kernel, the same sequence for each of its roles:
// whole tiles in turn (tile c, c + G, ...) for the full rounds; the tiles of the last round, which
// would leave some CTAs idle, are (for the adding epilogue) shared out in equal runs of
// (tile, k block) units, so a CTA may take the end of one tile and the beginning of the next, and
// the pieces of a tile meet in the float32 matrix they are added into.
struct Pieces {
    int nkb, tile, tile_end, step;
    long long u, u_end;
    // ``me`` of ``workers`` (CTAs, or pairs of CTAs) that share the tiles out
    __device__ Pieces(int n_tiles, int nkb_, int share_tail, int me, int workers) : nkb(nkb_) {
        step = workers;
        tile = me;
        tile_end = share_tail ? (n_tiles / step) * step : n_tiles;       // tiles of the full rounds
        const long long units = (long long)(n_tiles - tile_end) * nkb;
        u = (long long)tile_end * nkb + units * me / workers;
        u_end = (long long)tile_end * nkb + units * (me + 1) / workers;
    }
    __device__ bool next(int& t, int& kb0, int& kb1) {
        if (tile < tile_end) {
            t = tile; kb0 = 0; kb1 = nkb;
            tile += step;
            return true;
        }
        if (u >= u_end) return false;
        t = (int)(u / nkb);
        kb0 = (int)(u % nkb);
        kb1 = (int)min((long long)nkb, kb0 + (u_end - u));
        u += kb1 - kb0;
        return true;
    }
};

template <int BN, int EPI>
struct SmemP {
    static constexpr int A_BYTES = BM * BK * 2;
    static constexpr int B_BYTES = BN * BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES * (EPI == EPI_SWIGLU ? 2 : 1) + B_BYTES;
    static constexpr int STAGES = (196 * 1024) / STAGE_BYTES;
    static constexpr int XCH_BYTES = EPI == EPI_SWIGLU_IL ? 64 * 16 * 4 : 0;
    static constexpr int TOTAL = STAGES * STAGE_BYTES + 1024 + 256 + XCH_BYTES;
    static constexpr int ACC_COLS = BN * (EPI == EPI_SWIGLU ? 2 : 1);
    static constexpr int TMEM_COLS = 2 * ACC_COLS <= 32 ? 32 : 2 * ACC_COLS <= 64 ? 64 : 2 * ACC_COLS <= 128 ? 128
                                     : 2 * ACC_COLS <= 256 ? 256 : 512;
    static_assert(2 * ACC_COLS <= 512, "two accumulators must fit tensor memory");
};

template <int BN, int EPI, typename TO>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tc_persistent_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_w2,
                          const __grid_constant__ CUtensorMap map_a, GemmParams p) {
    using S = SmemP<BN, EPI>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* full = (uint64_t*)(smem + S::STAGES * S::STAGE_BYTES);
    uint64_t* empty = full + S::STAGES;
    uint64_t* acc_full = empty + S::STAGES;            // [2]
    uint64_t* acc_empty = acc_full + 2;                // [2]
    uint32_t* tmem_slot = (uint32_t*)(acc_empty + 2);
    volatile int* err = (volatile int*)(tmem_slot + 1);
    float* xch = (float*)(smem + S::STAGES * S::STAGE_BYTES + 256);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_w = (p.N + BM - 1) / BM, tiles_t = (p.T + BN - 1) / BN;
    const int n_tiles = tiles_w * tiles_t;
    const int nkb = (p.K + BK - 1) / BK;
    // token tiles vary fastest in the numbering of tiles, so the CTAs that run together share weight
    // tiles through the L2

    if (threadIdx.x == 0) {
        for (int s = 0; s < S::STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 4); }
        *err = 0;
        fence_barrier_init();
    }
    if (warp == 1) { tmem_alloc(tmem_slot, S::TMEM_COLS); tmem_relinquish(); }
    if (warp == 0 && lane == 0) {
        prefetch_tmap(&map_w); prefetch_tmap(&map_a);
        if (EPI == EPI_SWIGLU) prefetch_tmap(&map_w2);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_trigger();

    if (warp == 0) {
        if (lane == 0) {
            // the weights of the first stages depend on no kernel before this one: asked for before the wait
            long long pre = 0;
            {
                Pieces first(n_tiles, nkb, p.share_tail, blockIdx.x, gridDim.x);
                int tile, kb0, kb1;
                while (pre < S::STAGES && first.next(tile, kb0, kb1)) {
                    const int n0 = (tile / tiles_t) * BM;
                    for (int kb = kb0; kb < kb1 && pre < S::STAGES; ++kb, ++pre) {
                        uint8_t* st = smem + (int)pre * S::STAGE_BYTES;
                        mbar_expect_tx(&full[pre], S::STAGE_BYTES);
                        tma_load_2d(st, &map_w, &full[pre], kb * BK, n0);
                        if (EPI == EPI_SWIGLU) tma_load_2d(st + S::A_BYTES, &map_w2, &full[pre], kb * BK, n0);
                    }
                }
            }
            pdl_wait();
            long long it = 0;                            // stages filled so far, over all tiles
            bool ok = true;
            Pieces pieces(n_tiles, nkb, p.share_tail, blockIdx.x, gridDim.x);
            int tile, kb0, kb1;
            while (ok && pieces.next(tile, kb0, kb1)) {
                const int n0 = (tile / tiles_t) * BM, t0 = (tile % tiles_t) * BN;
                for (int kb = kb0; kb < kb1; ++kb, ++it) {
                    const int s = (int)(it % S::STAGES);
                    const uint32_t ph = (uint32_t)((it / S::STAGES) & 1);
                    uint8_t* st = smem + s * S::STAGE_BYTES;
                    if (it >= pre) {
                        ok = mbar_wait(&empty[s], ph ^ 1, err);
                        if (!ok) break;
                        mbar_expect_tx(&full[s], S::STAGE_BYTES);
                        tma_load_2d(st, &map_w, &full[s], kb * BK, n0);
                        if (EPI == EPI_SWIGLU) tma_load_2d(st + S::A_BYTES, &map_w2, &full[s], kb * BK, n0);
                    }
                    tma_load_2d(st + S::A_BYTES * (EPI == EPI_SWIGLU ? 2 : 1), &map_a, &full[s], kb * BK, t0);
                }
            }
            if (*err) {
                for (long long j = it > S::STAGES ? it - S::STAGES : 0; j < it; ++j) {
                    const long long tstart = clock64();
                    while (!mbar_try_wait(&full[j % S::STAGES], (uint32_t)((j / S::STAGES) & 1)))
                        if (clock64() - tstart > WAIT_LIMIT_CYCLES / 8) break;
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc(BN);
            long long it = 0;
            bool ok = true;
            Pieces pieces(n_tiles, nkb, p.share_tail, blockIdx.x, gridDim.x);
            int tile, kb0, kb1;
            for (int i = 0; ok && pieces.next(tile, kb0, kb1); ++i) {
                const int buf = i & 1;
                ok = mbar_wait(&acc_empty[buf], (uint32_t)(((i >> 1) & 1) ^ 1), err);   // the epilogue has read it
                if (!ok) break;
                tc_fence_after();
                const uint32_t acc = tmem_base + buf * S::ACC_COLS;
                for (int kb = kb0; kb < kb1; ++kb, ++it) {
                    const int s = (int)(it % S::STAGES);
                    const uint32_t ph = (uint32_t)((it / S::STAGES) & 1);
                    ok = mbar_wait(&full[s], ph, err);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(smem + s * S::STAGE_BYTES);
                    const uint32_t b_addr = a_addr + S::A_BYTES * (EPI == EPI_SWIGLU ? 2 : 1);
                    const uint64_t da = make_desc(a_addr), db = make_desc(b_addr);
                    const uint64_t da2 = make_desc(a_addr + S::A_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        const uint64_t koff = (uint64_t)((k * UMMA_K * 2) >> 4);
                        const uint32_t accum = (kb > kb0 || k > 0) ? 1u : 0u;
                        tc_mma_bf16(acc, da + koff, db + koff, idesc, accum);
                        if (EPI == EPI_SWIGLU) tc_mma_bf16(acc + BN, da2 + koff, db + koff, idesc, accum);
                    }
                    tc_commit(&empty[s]);
                }
                if (ok) tc_commit(&acc_full[buf]);
            }
        }
    } else {
        const int q = warp & 3;
        pdl_wait();
        bool ok = true;
        Pieces pieces(n_tiles, nkb, p.share_tail, blockIdx.x, gridDim.x);
        int tile, kb0, kb1;
        for (int i = 0; ok && pieces.next(tile, kb0, kb1); ++i) {
            const int buf = i & 1;
            ok = mbar_wait(&acc_full[buf], (uint32_t)((i >> 1) & 1), err);
            if (!ok) break;
            tc_fence_after();
            epilogue_tile<BN, EPI, TO>(p, tmem_base + buf * S::ACC_COLS, q, lane, tile / tiles_t, (tile % tiles_t) * BN, 0, xch);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[buf]);  // four warps: the accumulator may be written again
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, S::TMEM_COLS);
    }
    if (threadIdx.x == 0 && *err) atomicExch(p.error, 1);
}

// ---------------------------------------------------------------------------------------
// The same again with two CTAs (two SMs) on one tile of 256 weight rows x 256 tokens
// (tcgen05 cta_group::2).  Each CTA loads its own 128 weight rows and its own 128 of the tokens;
// the leader's MMAs read both CTAs' shared memory, so a CTA moves 32 KB a k block where the
// one-CTA kernel moves 48 KB for the same arithmetic, and six stages fit instead of four.  Each
// CTA's tensor memory receives its own 128 weight rows of the result and its own epilogue warps
// write them out; the tile sharing of the adding epilogue is the same, by pairs.
// ---------------------------------------------------------------------------------------
template <int EPI>
struct SmemPair {
    static constexpr int BNC = 128;                      // tokens a CTA loads
    static constexpr int A_BYTES = BM * BK * 2;
    static constexpr int B_BYTES = BNC * BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int STAGES = (196 * 1024) / STAGE_BYTES;
    static constexpr int XCH_BYTES = EPI == EPI_SWIGLU_IL ? 64 * 16 * 4 : 0;
    static constexpr int TOTAL = STAGES * STAGE_BYTES + 1024 + 256 + XCH_BYTES;
    static constexpr int ACC_COLS = 2 * BNC;             // the pair's tokens
    static constexpr int TMEM_COLS = 512;                // two accumulators
};

template <int EPI, typename TO>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_a, GemmParams p) {
    static_assert(EPI != EPI_SWIGLU, "one accumulator a tile");
    using S = SmemPair<EPI>;
    constexpr int BN2 = 2 * S::BNC, BM2 = 2 * BM;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* full = (uint64_t*)(smem + S::STAGES * S::STAGE_BYTES);     // the leader's are used
    uint64_t* empty = full + S::STAGES;
    uint64_t* acc_full = empty + S::STAGES;            // [2]
    uint64_t* acc_empty = acc_full + 2;                // [2], the leader's are used
    uint32_t* tmem_slot = (uint32_t*)(acc_empty + 2);
    volatile int* err = (volatile int*)(tmem_slot + 1);
    float* xch = (float*)(smem + S::STAGES * S::STAGE_BYTES + 256);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rank = (int)cluster_cta_rank();
    const bool leader = rank == 0;
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    const int tiles_w = (p.N + BM2 - 1) / BM2, tiles_t = (p.T + BN2 - 1) / BN2;
    const int n_tiles = tiles_w * tiles_t;
    const int nkb = (p.K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < S::STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 8); }   // 4 warps of each CTA
        *err = 0;
        fence_barrier_init();
    }
    if (warp == 1) { tmem_alloc_pair(tmem_slot, S::TMEM_COLS); tmem_relinquish_pair(); }
    if (warp == 0 && lane == 0) { prefetch_tmap(&map_w); prefetch_tmap(&map_a); }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();                                  // the other CTA's barriers exist before anything lands on them
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // No part in dependent launches: this kernel is launched the ordinary way and lets no kernel
    // start before it has ended (pairs of SMs are handed out whole, and with kernels that start
    // early in the mix the device was seen to stop making progress).

    if (warp == 0) {
        if (lane == 0) {
            long long it = 0;
            bool ok = true;
            Pieces pieces(n_tiles, nkb, p.share_tail, pair, n_pairs);
            int tile, kb0, kb1;
            while (ok && pieces.next(tile, kb0, kb1)) {
                const int n0 = (tile / tiles_t) * BM2 + rank * BM, t0 = (tile % tiles_t) * BN2 + rank * S::BNC;
                for (int kb = kb0; kb < kb1; ++kb, ++it) {
                    const int s = (int)(it % S::STAGES);
                    const uint32_t ph = (uint32_t)((it / S::STAGES) & 1);
                    ok = mbar_wait(&empty[s], ph ^ 1, err);
                    if (!ok) break;
                    uint8_t* st = smem + s * S::STAGE_BYTES;
                    if (leader) mbar_expect_tx(&full[s], 2 * S::STAGE_BYTES);      // both CTAs' copies
                    tma_load_2d_pair(st, &map_w, &full[s], kb * BK, n0);
                    tma_load_2d_pair(st + S::A_BYTES, &map_a, &full[s], kb * BK, t0);
                }
            }
            if (*err && leader) {
                for (long long j = it > S::STAGES ? it - S::STAGES : 0; j < it; ++j) {
                    const long long tstart = clock64();
                    while (!mbar_try_wait(&full[j % S::STAGES], (uint32_t)((j / S::STAGES) & 1)))
                        if (clock64() - tstart > WAIT_LIMIT_CYCLES / 8) break;
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && leader) {
            constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN2 >> 3) << 17) | ((uint32_t)(BM2 >> 4) << 24);
            long long it = 0;
            bool ok = true;
            Pieces pieces(n_tiles, nkb, p.share_tail, pair, n_pairs);
            int tile, kb0, kb1;
            for (int i = 0; ok && pieces.next(tile, kb0, kb1); ++i) {
                const int buf = i & 1;
                ok = mbar_wait(&acc_empty[buf], (uint32_t)(((i >> 1) & 1) ^ 1), err);   // both epilogues have read it
                if (!ok) break;
                tc_fence_after();
                const uint32_t acc = tmem_base + buf * S::ACC_COLS;
                for (int kb = kb0; kb < kb1; ++kb, ++it) {
                    const int s = (int)(it % S::STAGES);
                    const uint32_t ph = (uint32_t)((it / S::STAGES) & 1);
                    ok = mbar_wait(&full[s], ph, err);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(smem + s * S::STAGE_BYTES);
                    const uint64_t da = make_desc(a_addr), db = make_desc(a_addr + S::A_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        const uint64_t koff = (uint64_t)((k * UMMA_K * 2) >> 4);
                        tc_mma_bf16_pair(acc, da + koff, db + koff, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
                    }
                    tc_commit_pair(&empty[s]);           // frees the stage in both CTAs
                }
                if (ok) tc_commit_pair(&acc_full[buf]);  // wakes both epilogues
            }
        }
    } else {
        const int q = warp & 3;
        bool ok = true;
        Pieces pieces(n_tiles, nkb, p.share_tail, pair, n_pairs);
        int tile, kb0, kb1;
        for (int i = 0; ok && pieces.next(tile, kb0, kb1); ++i) {
            const int buf = i & 1;
            ok = mbar_wait(&acc_full[buf], (uint32_t)((i >> 1) & 1), err);
            if (!ok) break;
            tc_fence_after();
            epilogue_tile<BN2, EPI, TO>(p, tmem_base + buf * S::ACC_COLS, q, lane, (tile / tiles_t) * 2 + rank,
                                        (tile % tiles_t) * BN2, 0, xch);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_leader(&acc_empty[buf]);
        }
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();                                  // neither CTA's tensor or shared memory goes while the other may touch it
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, S::TMEM_COLS);
    }
    if (threadIdx.x == 0 && *err) atomicExch(p.error, 1);
}

// ---------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------
static EncodeTiledFn g_encode = nullptr;
static int load_encode() {
    if (!g_encode) g_encode = tensor_map_encoder();
    return g_encode ? 0 : UB_ERR_UNSUPPORTED;
}

// A tensor map of a row-major bfloat16 matrix [rows, cols] with row stride ld (elements): boxes
// of box_rows x 64 columns, 128-byte swizzle, zeros outside.  ``out_map`` is 128 bytes on the host.
UB_API int ub_tmap_bf16_2d(void* out_map, const void* base, long long rows, long long cols, long long ld, int box_rows) {
    if (load_encode()) return UB_ERR_UNSUPPORTED;
    if (((uintptr_t)base & 15) || (ld * 2) % 16 != 0 || box_rows < 1 || box_rows > 256 || rows < 1 || cols < 1) return UB_ERR_ARG;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = g_encode((CUtensorMap*)out_map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (void*)base, dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : UB_ERR_ARG;
}

static int g_use_pdl = 1;
UB_API void ub_gemm_tc_set_pdl(int on) { g_use_pdl = on ? 1 : 0; }

static int g_sm_count = 0;
static int sm_count() {
    if (!g_sm_count) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&g_sm_count, cudaDevAttrMultiProcessorCount, dev);
        if (g_sm_count <= 0) g_sm_count = 148;
    }
    return g_sm_count;
}

template <typename Kern>
static int launch_cfg(Kern kern, dim3 grid, int smem, const CUtensorMap* mw, const CUtensorMap* mw2, const CUtensorMap* ma,
                      const GemmParams& p, cudaStream_t st) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(NUM_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_use_pdl ? 1 : 0;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, *mw, *mw2, *ma, p);
    return e == cudaSuccess ? 0 : (int)e;
}

static int g_use_persistent = 1;
static int g_share_tail = 1;
UB_API void ub_gemm_tc_set_share_tail(int on) { g_share_tail = on ? 1 : 0; }
UB_API void ub_gemm_tc_set_persistent(int on) { g_use_persistent = on ? 1 : 0; }

template <int BN, int EPI, typename TO>
static int launch_one(const CUtensorMap* mw, const CUtensorMap* mw2, const CUtensorMap* ma, const GemmParams& p,
                      int splits, cudaStream_t st) {
    const int tiles = ((p.N + BM - 1) / BM) * ((p.T + BN - 1) / BN);
    if constexpr (BN >= 128) {
        // many tiles, K whole: CTAs that stay and overlap one tile's epilogue with the next tile's MMAs
        if (g_use_persistent && splits == 1 && tiles > sm_count()) {
            using SP = SmemP<BN, EPI>;
            GemmParams pp = p;
            pp.share_tail = (EPI == EPI_ADD && g_share_tail && tiles % sm_count() != 0) ? 1 : 0;
            static bool attr_p = false;
            auto kp = gemm_tc_persistent_kernel<BN, EPI, TO>;
            if (!attr_p) {
                cudaError_t e = cudaFuncSetAttribute(kp, cudaFuncAttributeMaxDynamicSharedMemorySize, SP::TOTAL);
                if (e != cudaSuccess) return (int)e;
                attr_p = true;
            }
            return launch_cfg(kp, dim3(sm_count()), SP::TOTAL, mw, mw2, ma, pp, st);
        }
    }
    using S = Smem<BN, EPI>;
    static bool attr_done = false;
    auto kern = gemm_tc_kernel<BN, EPI, TO>;
    if (!attr_done) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
        if (e != cudaSuccess) return (int)e;
        attr_done = true;
    }
    dim3 grid((p.N + BM - 1) / BM, (p.T + BN - 1) / BN, splits);
    if (grid.y > 65535 || grid.z > 65535) return UB_ERR_ARG;
    return launch_cfg(kern, grid, S::TOTAL, mw, mw2, ma, p, st);
}

template <int BN>
static int launch_bn(const CUtensorMap* mw, const CUtensorMap* mw2, const CUtensorMap* ma, const GemmParams& p,
                     int epi, int o_dtype, int splits, cudaStream_t st) {
    if (epi == EPI_STORE && o_dtype == UB_BF16) return launch_one<BN, EPI_STORE, __nv_bfloat16>(mw, mw2, ma, p, splits, st);
    if (epi == EPI_STORE && o_dtype == UB_F32) return launch_one<BN, EPI_STORE, float>(mw, mw2, ma, p, splits, st);
    if (epi == EPI_ADD && o_dtype == UB_F32) return launch_one<BN, EPI_ADD, float>(mw, mw2, ma, p, splits, st);
    if (epi == EPI_SWIGLU && o_dtype == UB_BF16) {
        if constexpr (BN <= 128) return launch_one<BN, EPI_SWIGLU, __nv_bfloat16>(mw, mw2, ma, p, splits, st);
        else return UB_ERR_ARG;
    }
    if (epi == EPI_SWIGLU_IL && o_dtype == UB_BF16) return launch_one<BN, EPI_SWIGLU_IL, __nv_bfloat16>(mw, mw2, ma, p, splits, st);
    return UB_ERR_UNSUPPORTED;
}

// map_w (and map_w2 for EPI_SWIGLU): weights [N, K], boxes of 128 rows; map_a: activations [T, K],
// boxes of ``bn`` rows.  splits > 1 cuts K into slices of kb_per_split blocks of 64: EPI_ADD then adds
// with atomics, EPI_STORE (float32 only) writes slice z at out + z * split_stride.
UB_API int ub_gemm_tc(const void* map_w, const void* map_w2, const void* map_a, void* out, int o_dtype, long long ldo,
                      long long split_stride, int T, int N, int K, int bn, int epi, int splits, int* error,
                      cudaStream_t st) {
    if (T <= 0 || N <= 0) return 0;
    if (K <= 0 || splits < 1) return UB_ERR_ARG;
    if (splits > 1 && (epi == EPI_SWIGLU || epi == EPI_SWIGLU_IL)) return UB_ERR_ARG;
    if (epi == EPI_SWIGLU_IL && (N % 128) != 0) return UB_ERR_ARG;
    if (splits > 1 && epi == EPI_STORE && o_dtype != UB_F32) return UB_ERR_ARG;
    const int nkb = (K + BK - 1) / BK;
    GemmParams p;
    p.out = out; p.ldo = ldo; p.split_stride = splits > 1 ? split_stride : 0;
    p.T = T; p.N = N; p.K = K;
    p.kb_per_split = (nkb + splits - 1) / splits;
    p.atomic = (epi == EPI_ADD && splits > 1) ? 1 : 0;
    p.share_tail = 0;
    p.error = error;
    if ((long long)(splits - 1) * p.kb_per_split >= nkb) return UB_ERR_ARG;      // an empty slice
    const CUtensorMap* mw = (const CUtensorMap*)map_w;
    const CUtensorMap* mw2 = (const CUtensorMap*)(map_w2 ? map_w2 : map_w);
    const CUtensorMap* ma = (const CUtensorMap*)map_a;
    switch (bn) {
        case 16: return launch_bn<16>(mw, mw2, ma, p, epi, o_dtype, splits, st);
        case 32: return launch_bn<32>(mw, mw2, ma, p, epi, o_dtype, splits, st);
        case 64: return launch_bn<64>(mw, mw2, ma, p, epi, o_dtype, splits, st);
        case 128: return launch_bn<128>(mw, mw2, ma, p, epi, o_dtype, splits, st);
        case 256: return launch_bn<256>(mw, mw2, ma, p, epi, o_dtype, splits, st);
    }
    return UB_ERR_ARG;
}

// The two-CTA kernel: many tokens (T > 128), K whole.  map_w: boxes of 128 weight rows; map_a: boxes
// of 128 tokens.  Epilogues: store, add (float32 out), interleaved gate product.
template <int EPI, typename TO>
static int launch_pair(const CUtensorMap* mw, const CUtensorMap* ma, GemmParams p, cudaStream_t st) {
    using S = SmemPair<EPI>;
    auto kern = gemm_tc_pair_kernel<EPI, TO>;
    static bool attr_done = false;
    if (!attr_done) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
        if (e != cudaSuccess) return (int)e;
        attr_done = true;
    }
    const int n_pairs = sm_count() / 2;
    const int tiles = ((p.N + 2 * BM - 1) / (2 * BM)) * ((p.T + 255) / 256);
    p.share_tail = (EPI == EPI_ADD && g_share_tail && tiles % n_pairs != 0 && tiles > n_pairs) ? 1 : 0;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * (tiles < n_pairs ? tiles : n_pairs));
    cfg.blockDim = dim3(NUM_THREADS);
    cfg.dynamicSmemBytes = S::TOTAL;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;                  // not a programmatic dependent of the kernel before it
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, *mw, *ma, p);
    return e == cudaSuccess ? 0 : (int)e;
}

UB_API int ub_gemm_tc_pair(const void* map_w, const void* map_a, void* out, int o_dtype, long long ldo, int T, int N,
                           int K, int epi, int* error, cudaStream_t st) {
    if (T <= 0 || N <= 0) return 0;
    if (K <= 0) return UB_ERR_ARG;
    if (epi == EPI_SWIGLU_IL && (N % 128) != 0) return UB_ERR_ARG;
    GemmParams p;
    p.out = out; p.ldo = ldo; p.split_stride = 0;
    p.T = T; p.N = N; p.K = K;
    p.kb_per_split = (K + BK - 1) / BK;
    p.atomic = 0; p.share_tail = 0; p.error = error;
    const CUtensorMap* mw = (const CUtensorMap*)map_w;
    const CUtensorMap* ma = (const CUtensorMap*)map_a;
    if (epi == EPI_STORE && o_dtype == UB_BF16) return launch_pair<EPI_STORE, __nv_bfloat16>(mw, ma, p, st);
    if (epi == EPI_STORE && o_dtype == UB_F32) return launch_pair<EPI_STORE, float>(mw, ma, p, st);
    if (epi == EPI_ADD && o_dtype == UB_F32) return launch_pair<EPI_ADD, float>(mw, ma, p, st);
    if (epi == EPI_SWIGLU_IL && o_dtype == UB_BF16) return launch_pair<EPI_SWIGLU_IL, __nv_bfloat16>(mw, ma, p, st);
    return UB_ERR_UNSUPPORTED;
}
