// A decode step's whole stack of layers as ONE resident kernel: one CTA an SM, all of them alive
// from the first layer to the last, running a program of phases that the host wrote into global
// memory (norm, product, attention, merge of the key slices, gate product).  Compiled for one
// head size (-DHEAD_DIM=64 or 128); one new token a sequence, at most 64 sequences.
//
// Why: run as separate kernels, a layer's attention block is a chain of six short kernels that wait
// for one another, and while they do the memory is idle except for what the next product's ring of
// shared memory holds.  Here one warp of every CTA loads weights and cache pages into one ring of
// shared-memory slots for the WHOLE program, phase after phase, held back only by free slots: what
// it loads (weights; cache pages of earlier steps) depends on no phase.  The warps that compute go
// through the phases in order and meet all other CTAs at a barrier in global memory after each; while
// they wait there, or for a phase's short latency-bound start, the ring keeps filling, so the memory
// works for as long as the program has bytes left to read.
//
// Roles in a CTA (192 threads): warp 0 loads (TMA), warp 1 issues tcgen05 MMAs, warps 2-5 are the
// workers: epilogues of the products, attention arithmetic (mma.sync, as in attn_mma.cu), and the
// row-wise phases.  Every product is cut into (256 weight rows, 64 k columns) units (two accumulators
// of 128 lanes fed by one token tile) that are dealt
// out evenly and contiguously to the CTAs; a CTA adds its partial tiles into a float32 matrix with
// red.global.add (the residual stream itself for the output and down projections, a cleared scratch
// matrix for q/k/v and gate/up).  Attention is cut the same way: its units are (sequence, kv head,
// page), a CTA's run of pages of one (sequence, kv head) gives a partial result, and a merge phase
// puts the partial results together.  Every wait has a time limit and raises a flag.
//
// The loading warp is one thread that has to hand out a 32 KB unit every 0.7 us to keep the memory busy,
// so its loop holds no division, no record read from global memory and no local array (each cost it the
// better part of a microsecond a turn), and it asks a barrier with test_wait, which returns at once.
//
// Measured, this kernel is slower than the separate kernels (see kernels/decode_stack.py): the grid
// barriers (nine a layer, 2-3 us each) and the short phases between them outweigh what the ring saves.
// It is kept as an alternative that is switched on by hand.
//
// The arithmetic is the same as the separate kernels': rmsnorm.cpp:10-17, qwen_block.cpp:682-690,
// :713-727, :94-135, :775-783, :165-182 of the reference, restated for a ragged batch of one token each.
#include "attn_device.cuh"
#include <string.h>

static_assert(HEAD_DIM == 64 || HEAD_DIM == 128, "the layer-stack kernel is built for head sizes 64 and 128");

enum : int { PH_NORM = 0, PH_GEMM = 1, PH_ATTN = 2, PH_MERGE = 3, PH_SILU = 4 };

// One phase of the program.  Which fields a phase reads is said beside its type; pointers that are
// null mean "the residual stream of this launch" where noted.
struct Phase {
    int type;
    int pad0;
    // PH_GEMM: out[t, n] += sum_k act[t, k] w[n, k]; act through tensor map map_b (bfloat16 [BN, K], boxes of BN rows),
    //          w through map_w ([N, K], boxes of 128 rows); out float32 [T, ldo] (null: the residual stream)
    int map_w, map_b, N, K;
    float* out;
    long long ldo;
    // PH_NORM: h[t, :] = bf16(x[t, :] * w * inv_rms(x[t, :])), x the residual stream [T, width]; clears zero[0 .. zero_n)
    const float* w;
    bf16* h;
    int width;
    float eps;
    float* zero;
    long long zero_n;
    // PH_SILU: act[t, 64 b + j] = bf16(silu(gu[t, 128 b + j]) * gu[t, 128 b + 64 + j]), gu float32 [T, 2 F]
    const float* gu;
    bf16* act;
    int F, pad1;
    // PH_ATTN: q, k, v of the step from qkv float32 [T, (nh + 2 nkv) HD] (sums complete); per-head norm with qw, kw
    //          (null: none), rotation by cs, sn [positions, HD / 2] (null: none); the new key and value go into
    //          kcache, vcache (null: the cache is another run's) and into the loaded page; keys and values through
    //          map_k, map_v; partial results (per segment) to part_o [segments, 16, HD], part_ml [segments, 16, 2]
    // PH_MERGE: o[t, head, :] = merge of the segments of (sequence t, kv head of head); same fields
    const float* qkv;
    const float* qw; const float* kw; const float* cs; const float* sn;
    bf16* kcache; bf16* vcache;
    float* part_o; float* part_ml;
    bf16* o;
    int nh, nkv, window, ring, pages_per_seq, map_k, map_v, table;     // table: which of the launch's page tables
    float c;                      // scale * log2(e)
    int pad2;
};

// The program's tensor maps travel in the kernel's parameters: there the TMA unit finds them as it finds
// those of the other kernels (maps read from global memory made every copy wait for its descriptor).
constexpr int MAX_MAPS = 224;
struct MapPack { CUtensorMap m[MAX_MAPS]; };

struct StackParams {
    const Phase* phases; int n_phases;
    int T;                                 // tokens = sequences of the step
    float* x;                              // residual stream float32 [T, width]
    const int* seq_before;                 // positions of the step's tokens
    const int* tables[4];                  // page tables of the cache's groups
    int window_b;                          // the one window (besides "none") that phases of this program use, or 0
    unsigned int* counter;                 // the barrier between phases: cleared by the host before the launch
    int* error;
    long long* trace;                      // null, or [n_phases + 1]: when CTA 0 began each phase and ended the last (ns)
};

constexpr int SK_THREADS = 192;
constexpr int W_ROWS = 256;                 // weight rows of a unit: two accumulators of 128 lanes
constexpr int W_BYTES = W_ROWS * 64 * 2;    // a unit's weights (256 rows of a k block); a key page and a value page fit there too
constexpr int BKK = 64;
constexpr int MAX_SEQS = 64;

template <int BN>
struct SK {
    static constexpr int SLOT = W_BYTES + BN * 128;
    static constexpr int QS_BYTES = 16 * LDS * 2;
    static constexpr int RED_BYTES = 64 * (HD + 2) * 4;
    static constexpr int TAB_BYTES = 2 * (MAX_SEQS + 1) * 4 + 2 * MAX_SEQS * 4 * 2;     // cum, pages and first tile, for two windows
    static constexpr int FIXED = QS_BYTES + RED_BYTES + TAB_BYTES + 1024 /*barriers, words*/ + 1024 /*alignment*/;
    static constexpr int SLOTS_RAW = (227 * 1024 - FIXED) / SLOT;
    static constexpr int SLOTS = SLOTS_RAW > 12 ? 12 : SLOTS_RAW;
    static constexpr int TOTAL = SLOTS * SLOT + FIXED;
    static_assert(SLOTS >= 3, "ring too short");
    static_assert(2 * PAGE_BYTES <= W_BYTES, "a key page and a value page share a slot");
};

__device__ __forceinline__ unsigned ld_acquire(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }
__device__ __forceinline__ void fence_tensormap(const CUtensorMap* m) {
    asm volatile("fence.proxy.tensormap::generic.acquire.gpu [%0], 128;" ::"l"(m) : "memory");
}
// FE neighbouring floats that another CTA wrote in an earlier phase: from the L2, never from this SM's L1
__device__ __forceinline__ void ldcg_vec(const float* p, float* v) {
    if constexpr (FE == 4) { const float4 t = __ldcg(reinterpret_cast<const float4*>(p)); v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w; }
    else { const float2 t = __ldcg(reinterpret_cast<const float2*>(p)); v[0] = t.x; v[1] = t.y; }
}
__device__ __forceinline__ long long global_ns() {
    long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void named_sync(int id, int n) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(n) : "memory"); }

// units dealt out evenly and contiguously: CTA c of G takes [begin(c), begin(c + 1))
__device__ __forceinline__ long long deal_begin(long long U, int c, int G) { return (U * c) / G; }
__device__ __forceinline__ int deal_owner(long long g, long long U, int G) {
    int c = (int)((g * G) / U);
    if (c >= G) c = G - 1;
    while (c + 1 < G && deal_begin(U, c + 1, G) <= g) ++c;
    while (c > 0 && deal_begin(U, c, G) > g) --c;
    return c;
}

// What the sequences' lengths make of an attention phase: pages a sequence's keys span (np), the
// first of them (tf), and running sums (cum).  Two tables: no window, and the program's one window.
struct SeqTables {
    int* cum;       // [2][MAX_SEQS + 1]
    int* np;        // [2][MAX_SEQS]
    int* tf;        // [2][MAX_SEQS]
};
__device__ __forceinline__ int table_of(int window) { return window > 0 ? 1 : 0; }

// units of an attention phase: (sequence, kv head, page); all kv heads of a sequence have the same pages
__device__ __forceinline__ long long attn_units(const SeqTables& t, int which, int T, int nkv) {
    return (long long)t.cum[which * (MAX_SEQS + 1) + T] * nkv;
}
__device__ __forceinline__ void attn_locate(const SeqTables& t, int which, int T, int nkv, long long g, int& seq, int& kvh, int& j) {
    const int* cum = t.cum + which * (MAX_SEQS + 1);
    int lo = 0, hi = T - 1;
    while (lo < hi) {                                   // the last sequence whose first unit is at or before g
        const int mid = (lo + hi + 1) >> 1;
        if ((long long)cum[mid] * nkv <= g) lo = mid; else hi = mid - 1;
    }
    seq = lo;
    const long long r = g - (long long)cum[lo] * nkv;
    const int n = t.np[which * MAX_SEQS + lo];
    kvh = (int)(r / n);
    j = (int)(r % n);
}

template <int BN>
__global__ void __launch_bounds__(SK_THREADS, 1) decode_stack_kernel(const __grid_constant__ StackParams sp,
                                                                     const __grid_constant__ MapPack maps) {
    using S = SK<BN>;
    constexpr int NS = S::SLOTS;
    constexpr int TMEM_COLS = 4 * BN < 32 ? 32 : 4 * BN;           // two accumulator buffers of two halves
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* ring = smem;                                           // [NS][SLOT]: weights | tokens, or a page
    bf16* Qs = (bf16*)(ring + NS * S::SLOT);                        // [16][LDS]
    float* red = (float*)((uint8_t*)Qs + S::QS_BYTES);              // [64][HD + 2]
    int* tab = (int*)((uint8_t*)red + S::RED_BYTES);
    SeqTables st{tab, tab + 2 * (MAX_SEQS + 1), tab + 2 * (MAX_SEQS + 1) + 2 * MAX_SEQS};
    uint64_t* full = (uint64_t*)((uint8_t*)tab + S::TAB_BYTES);     // [NS]
    uint64_t* empty = full + NS;                                    // [NS] four arrivals free a slot: the four workers', or the
                                                                    //      MMA's commit and three arrivals of its thread
    uint64_t* acc_full = empty + NS;                                // [2]
    uint64_t* acc_empty = acc_full + 2;                             // [2]
    uint32_t* tmem_slot = (uint32_t*)(acc_empty + 2);
    volatile int* err = (volatile int*)(tmem_slot + 1);
    float* scratch = (float*)(tmem_slot + 4);                       // [8] for the workers' row sums

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int c = blockIdx.x, G = gridDim.x;
    const int T = sp.T;

    if (threadIdx.x == 0) {
        for (int s = 0; s < NS; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 4); }
        for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 4); }
        *err = 0;
        fence_barrier_init();
    }
    if (warp == 1) { tmem_alloc(tmem_slot, TMEM_COLS); tmem_relinquish(); }
    // the sequences' page ranges, without a window and with the program's one window
    for (int i = threadIdx.x; i < 2 * MAX_SEQS; i += SK_THREADS) {
        const int which = i / MAX_SEQS, s = i % MAX_SEQS;
        int n = 0, first = 0;
        if (s < T) {
            const int pos = sp.seq_before[s];
            const int w = which ? sp.window_b : 0;
            first = (which && w > 0) ? max(0, pos - w + 1) / KT : 0;
            n = pos / KT - first + 1;
        }
        st.np[which * MAX_SEQS + s] = n;
        st.tf[which * MAX_SEQS + s] = first;
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (threadIdx.x < 2) {
        int* cum = st.cum + threadIdx.x * (MAX_SEQS + 1);
        int a = 0;
        for (int s = 0; s < MAX_SEQS; ++s) { cum[s] = a; a += st.np[threadIdx.x * MAX_SEQS + s]; }
        cum[MAX_SEQS] = a;
        // sequences past T have no pages, so cum[T] is the total as well
    }
    __syncthreads();
    const uint32_t tmem_base = *tmem_slot;

    // How many ring slots a CTA's share of a phase takes: the same count for every role, which is how
    // the loading warp, the MMA warp and the workers stay on the same slot without talking.
    auto phase_units = [&](const Phase& ph) -> long long {
        if (ph.type == PH_GEMM) return (long long)((ph.N + W_ROWS - 1) / W_ROWS) * ((ph.K + BKK - 1) / BKK);
        if (ph.type == PH_ATTN) return attn_units(st, table_of(ph.window), T, ph.nkv);
        return 0;
    };

    // the barrier between phases: phase p may begin when every CTA has finished phase p - 1.  A thread
    // remembers how far it has seen the program open and looks at the counter only beyond that.
    int open_upto = 0;
    auto phase_open = [&](int p) -> bool {
        if (p <= open_upto) return true;
        const unsigned done = ld_acquire(sp.counter) / (unsigned)G;       // phases every CTA has finished
        if ((int)done > open_upto) open_upto = (int)done;
        return p <= open_upto;
    };
    // one lane a warp watches the counter; after an error nothing waits any more
    auto wait_phase = [&](int p) -> bool {
        int good = 1;
        if (lane == 0 && !phase_open(p)) {
            const long long t0 = clock64();
            while (!phase_open(p)) {
                if (*err) { good = 0; break; }
                if (clock64() - t0 > WAIT_LIMIT_CYCLES) { *err = 1; good = 0; break; }
                __nanosleep(64);
            }
        }
        return __shfl_sync(0xffffffffu, good, 0) != 0;
    };

    if (warp == 0) {
        // ------------------------------------------------------------------------------------
        // the loading warp: two cursors over the program.  The first runs ahead as far as free slots
        // allow and loads what depends on no phase (weights, pages); the second follows and loads the
        // token tiles of products whose phase has opened, into the slots the first has set up.
        // ------------------------------------------------------------------------------------
        if (lane == 0) {
            // A cursor keeps its phase's record and its place in it (tile and k block of a product; sequence,
            // kv head and page of attention) and steps them; nothing is divided and no record is read from
            // global memory inside the loop, where either costs this one thread most of a microsecond a turn.
            struct Cur {
                int p, left, slot, n;                 // units left of this CTA's share; next ring slot; slots handed out so far
                int tile, kb, nkb;                    // product
                int seq, kvh, j, np, which;           // attention
                Phase ph;
            };
            Cur a, b;
            a.p = b.p = -1; a.left = b.left = 0; a.slot = b.slot = 0; a.n = b.n = 0;
            uint32_t used = 0, par = 0;            // a bit a slot: handed out before; parity its barrier will have passed when free again
            auto next_phase = [&](Cur& k) {
                for (++k.p; k.p < sp.n_phases; ++k.p) {
                    k.ph = sp.phases[k.p];
                    const Phase& ph = k.ph;
                    const long long U = phase_units(ph);
                    if (U <= 0) continue;
                    const long long u0 = deal_begin(U, c, G), u1 = deal_begin(U, c + 1, G);
                    if (u0 >= u1) continue;
                    k.left = (int)(u1 - u0);
                    if (ph.type == PH_GEMM) {
                        k.nkb = (ph.K + BKK - 1) / BKK;
                        k.tile = (int)(u0 / k.nkb); k.kb = (int)(u0 % k.nkb);
                    } else {
                        k.which = table_of(ph.window);
                        attn_locate(st, k.which, T, ph.nkv, u0, k.seq, k.kvh, k.j);
                        k.np = st.np[k.which * MAX_SEQS + k.seq];
                    }
                    return;
                }
            };
            auto step_slot = [&](Cur& k, int by) { k.n += by; k.slot += by; if (k.slot >= NS) k.slot -= NS; };
            next_phase(a);
            next_phase(b);
            int fenced_upto = -1, fenced_open = -1, look = 0;
            long long t_idle = -1;
            bool ok = true;
            while (ok && (a.p < sp.n_phases || b.p < sp.n_phases)) {
                bool moved = false;
                // ---- second cursor: token tiles of opened product phases
                if (b.p < sp.n_phases) {
                    const Phase& ph = b.ph;
                    if (ph.type == PH_ATTN) {                       // nothing to load here: its pages came with the first cursor
                        if (b.p < a.p || a.p >= sp.n_phases) {              // only once the first cursor is past it
                            b.n += b.left;
                            b.slot = (b.slot + b.left) % NS;
                            next_phase(b);
                            moved = true;
                        }
                    } else if (b.n < a.n && (b.p <= open_upto || (--look <= 0 && (look = 8, phase_open(b.p))))) {
                        if (b.p > fenced_open) { fence_proxy_async_all(); fenced_open = b.p; }   // other CTAs' stores of the tokens, before TMA reads them
                        const int s = b.slot;
                        tma_load_2d(ring + s * S::SLOT + W_BYTES, &maps.m[ph.map_b], &full[s], b.kb * BKK, 0);
                        step_slot(b, 1);
                        if (++b.kb == b.nkb) b.kb = 0;
                        if (--b.left == 0) next_phase(b);
                        moved = true;
                    }
                }
                // ---- first cursor: weights and pages, as far ahead as slots are free
                if (a.p < sp.n_phases) {
                    const Phase& ph = a.ph;
                    if (a.p > fenced_upto) {
                        if (ph.type == PH_GEMM) { prefetch_tmap(&maps.m[ph.map_w]); prefetch_tmap(&maps.m[ph.map_b]); }
                        else { prefetch_tmap(&maps.m[ph.map_k]); prefetch_tmap(&maps.m[ph.map_v]); }
                        fenced_upto = a.p;
                    }
                    const int s = a.slot;
                    if (!((used >> s) & 1u) || mbar_test_wait(&empty[s], (par >> s) & 1u)) {
                        if ((used >> s) & 1u) par ^= 1u << s;
                        used |= 1u << s;
                        if (ph.type == PH_GEMM) {
                            mbar_expect_tx(&full[s], W_BYTES + BN * 128);          // the tokens follow with the second cursor
                            tma_load_2d(ring + s * S::SLOT, &maps.m[ph.map_w], &full[s], a.kb * BKK, a.tile * W_ROWS);
                            step_slot(a, 1);
                            if (++a.kb == a.nkb) { a.kb = 0; ++a.tile; }
                        } else {
                            const int tile = st.tf[a.which * MAX_SEQS + a.seq] + a.j;
                            const int* table = sp.tables[ph.table];
                            const int page = table[(long long)a.seq * ph.pages_per_seq + ((tile * KT) % ph.ring) / KT];
                            const int r0 = (page * ph.nkv + a.kvh) * KT;
                            mbar_expect_tx(&full[s], 2 * PAGE_BYTES);
                            for (int kv = 0; kv < 2; ++kv)
                                for (int nb = 0; nb < NBLK; ++nb)
                                    tma_load_2d(ring + s * S::SLOT + kv * PAGE_BYTES + nb * BLK_BYTES, &maps.m[kv ? ph.map_v : ph.map_k], &full[s], nb * 64, r0);
                            step_slot(a, 1);
                            if (++a.j == a.np) {
                                a.j = 0;
                                if (++a.kvh == ph.nkv) { a.kvh = 0; ++a.seq; }
                                if (a.seq < T) a.np = st.np[a.which * MAX_SEQS + a.seq];
                            }
                        }
                        if (--a.left == 0) next_phase(a);
                        moved = true;
                    }
                }
                if (moved) { t_idle = -1; continue; }
                if (*err) { ok = false; break; }
                if (t_idle < 0) t_idle = clock64();
                else if (clock64() - t_idle > WAIT_LIMIT_CYCLES) { *err = 1; ok = false; }
            }
            if (*err) {
                // let copies in flight land before the CTA's memory goes away: every slot handed out and not
                // yet completed (a product's slot whose tokens never came cannot complete; its weights have
                // landed long before the limit of this wait)
                const long long tstart = clock64();
                for (int i = a.n > NS ? a.n - NS : 0; i < a.n; ++i)
                    while (!mbar_try_wait(&full[i % NS], (uint32_t)((i / NS) & 1))) if (clock64() - tstart > WAIT_LIMIT_CYCLES / 8) break;
            }
        }
    } else {
        // ------------------------------------------------------------------------------------
        // the MMA warp (1) and the workers (2-5) go through the phases in order
        // ------------------------------------------------------------------------------------
        const bool worker = warp >= 2;
        const int wq = warp & 3;                                   // which quarter of the 128 accumulator lanes a worker reads
        const int wt = (warp - 2) * 32 + lane;                     // 0..127 among the workers
        int n_used = 0;                                            // ring slots this CTA's earlier phases took
        int pieces = 0;                                            // accumulator uses so far (two buffers in turn)
        bool ok = true;
        // After an error (a wait that ran out) nothing is computed any more, but every thread still walks
        // the same phases and meets the same barriers inside the CTA, so that none is left waiting at one.
        for (int p = 0; p < sp.n_phases; ++p) {
            const Phase ph = sp.phases[p];                   // a copy: the loops below read its fields often
            if (!wait_phase(p)) ok = false;
            if (sp.trace && c == 0 && warp == 1 && lane == 0) sp.trace[p] = global_ns();
            if (ph.type == PH_GEMM) {
                const int nkb = (ph.K + BKK - 1) / BKK;
                const long long U = phase_units(ph);
                const int u0 = (int)deal_begin(U, c, G), u1 = (int)deal_begin(U, c + 1, G);
                const int tile0 = u0 / nkb, kb_first = u0 % nkb;
                float* out = ph.out ? ph.out : sp.x;
                if (warp == 1) {
                    if (lane == 0) {
                        constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
                        int s = n_used % NS;                              // the ring slot and its barrier's parity, stepped
                        uint32_t par = (uint32_t)((n_used / NS) & 1);
                        int pc = pieces;
                        for (int u = u0, kb0 = kb_first, tile = tile0; u < u1 && ok; kb0 = 0, ++tile) {
                            const int piece_end = min(u1, u - kb0 + nkb);
                            const int buf = pc & 1;
                            ok = mbar_wait(&acc_empty[buf], (uint32_t)(((pc >> 1) & 1) ^ 1), err);      // its last reader has finished
                            if (!ok) break;                                  // (this thread meets no barrier inside the phase)
                            tc_fence_after();
                            const uint32_t acc = tmem_base + buf * 2 * BN;     // the lower 128 weight rows; the upper at + BN
                            const bool upper = (long long)tile * W_ROWS + 128 < ph.N;      // (rows past N would be zeros: skipped)
                            bool first = true;
                            for (; u < piece_end; ++u) {
                                ok = mbar_wait(&full[s], par, err);
                                if (!ok) break;
                                tc_fence_after();
                                const uint32_t a_addr = smem_u32(ring + s * S::SLOT);
                                const uint64_t da = make_desc(a_addr), db = make_desc(a_addr + W_BYTES);
#pragma unroll
                                for (int k = 0; k < BKK / 16; ++k) {
                                    const uint64_t koff = (uint64_t)((k * 32) >> 4);
                                    tc_mma_bf16(acc, da + koff, db + koff, idesc, (first && k == 0) ? 0u : 1u);
                                }
                                if (upper) {
                                    const uint64_t da2 = make_desc(a_addr + 128 * 128);
#pragma unroll
                                    for (int k = 0; k < BKK / 16; ++k) {
                                        const uint64_t koff = (uint64_t)((k * 32) >> 4);
                                        tc_mma_bf16(acc + BN, da2 + koff, db + koff, idesc, (first && k == 0) ? 0u : 1u);
                                    }
                                }
                                first = false;
                                tc_commit(&empty[s]);
                                mbar_arrive(&empty[s]); mbar_arrive(&empty[s]); mbar_arrive(&empty[s]);     // (the commit is the fourth)
                                if (++s == NS) { s = 0; par ^= 1u; }
                            }
                            if (ok) tc_commit(&acc_full[buf]);
                            ++pc;
                        }
                    }
                } else {
                    int pc = pieces;
                    for (int u = u0, kb0 = kb_first, tile = tile0; u < u1 && ok; kb0 = 0, ++tile) {
                        const int piece_end = min(u1, u - kb0 + nkb);
                        const int buf = pc & 1;
                        ok = mbar_wait(&acc_full[buf], (uint32_t)((pc >> 1) & 1), err);
                        if (!ok) break;
                        tc_fence_after();
#pragma unroll 1
                        for (int half = 0; half < 2; ++half) {
                            const int n = tile * W_ROWS + half * 128 + wq * 32 + lane;
                            if (tile * W_ROWS + half * 128 >= ph.N) break;          // (no MMA wrote the upper half then)
#pragma unroll 1
                            for (int c0 = 0; c0 < BN; c0 += 16) {
                                if (c0 >= T) break;
                                uint32_t r[16];
                                tmem_ld16(tmem_base + ((uint32_t)(wq * 32) << 16) + (uint32_t)((buf * 2 + half) * BN + c0), r);
                                tmem_ld_wait();
                                if (n < ph.N) {
#pragma unroll
                                    for (int cc = 0; cc < 16; ++cc) {
                                        const int t = c0 + cc;
                                        if (t >= T) break;
                                        asm volatile("red.global.add.f32 [%0], %1;" ::"l"(out + (long long)t * ph.ldo + n), "f"(__uint_as_float(r[cc])) : "memory");
                                    }
                                }
                            }
                        }
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&acc_empty[buf]);
                        u = piece_end;
                        ++pc;
                    }
                }
                // both roles count the same pieces and slots
                if (u1 > u0) {
                    pieces += (u1 - 1) / nkb - tile0 + 1;
                    n_used += u1 - u0;
                }
            } else if (ph.type == PH_ATTN) {
                const int which = table_of(ph.window);
                const long long U = phase_units(ph);
                const long long u0 = deal_begin(U, c, G), u1 = deal_begin(U, c + 1, G);
                if (worker) {
                    const int Gq = ph.nh / ph.nkv;
                    const int heads_all = ph.nh + 2 * ph.nkv;
                    FusedQKV f{ph.qkv, 1, 0, ph.qw, ph.kw, ph.cs, ph.sn, 0.f, ph.kcache, ph.vcache};
                    f.eps = ph.eps;
                    const int* table = sp.tables[ph.table];
                    int sl = n_used % NS;                                 // the unit's slot: its key page, then its value page
                    uint32_t parl = (uint32_t)((n_used / NS) & 1);
                    for (long long u = u0; u < u1;) {
                        int seq, kvh, j;
                        attn_locate(st, which, T, ph.nkv, u, seq, kvh, j);
                        const int np_ = st.np[which * MAX_SEQS + seq], tf_ = st.tf[which * MAX_SEQS + seq];
                        const long long run_end = min(u1, u + (np_ - j));
                        const int n_run = (int)(run_end - u);
                        const int pos = sp.seq_before[seq];
                        const int t_last = pos / KT;
                        const bool has_new = ph.kcache != nullptr && tf_ + j + n_run - 1 == t_last;
                        const int new_row = pos % KT;
                        // ---- q of this kv head's group, and the new key and value where they are this run's
                        float co[FE], si[FE], gq[FE], gk[FE], new_k[FE], new_v[FE];
                        if (ph.cs) {
                            const int j0 = (lane & 15) * FE;
                            load_vec<float, FE>(ph.cs + (long long)pos * (HD / 2) + j0, co);
                            load_vec<float, FE>(ph.sn + (long long)pos * (HD / 2) + j0, si);
                        }
                        if (ph.qw) load_vec<float, FE>(ph.qw + lane * FE, gq);
                        if (ph.kw) load_vec<float, FE>(ph.kw + lane * FE, gk);
                        const float* trow = ph.qkv + (long long)seq * heads_all * HD;
                        const int w4 = warp - 2;
                        const bool mine = has_new && w4 == new_row / 16;
                        for (int r = w4; r < 16; r += 4) {
                            float v[FE];
                            if (r < Gq) {
                                ldcg_vec(trow + (long long)(kvh * Gq + r) * HD + lane * FE, v);
                                fused_finish(f, ph.qw ? gq : nullptr, ph.cs != nullptr, co, si, lane, v);
                            } else {
#pragma unroll
                                for (int i = 0; i < FE; ++i) v[i] = 0.f;
                            }
                            store_vec<bf16, FE>(Qs + r * LDS + lane * FE, v);
                        }
                        if (mine) {
                            ldcg_vec(trow + (long long)(ph.nh + kvh) * HD + lane * FE, new_k);
                            ldcg_vec(trow + (long long)(ph.nh + ph.nkv + kvh) * HD + lane * FE, new_v);
                            fused_finish(f, ph.kw ? gk : nullptr, ph.cs != nullptr, co, si, lane, new_k);
                            const PagedKV pc{table, ph.pages_per_seq, ph.ring, KT, ph.nkv, HD};
                            const long long at = paged_offset(pc, seq, pos, kvh) + lane * FE;
                            store_vec<bf16, FE>(ph.kcache + at, new_k);
                            store_vec<bf16, FE>(ph.vcache + at, new_v);
                        }
                        named_sync(1, 128);                               // q is whole before any warp reads it
                        float o[DTILES][4];
#pragma unroll
                        for (int dt = 0; dt < DTILES; ++dt) o[dt][0] = o[dt][1] = o[dt][2] = o[dt][3] = 0.f;
                        float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
                        int row_pos[2] = {pos, pos};
                        bool row_ok[2] = {(lane >> 2) < Gq, (lane >> 2) + 8 < Gq};
                        for (int i = 0; i < n_run; ++i) {
                            const int s_now = sl;
                            const uint32_t par_now = parl;
                            if (++sl == NS) { sl = 0; parl ^= 1u; }
                            if (ok) ok = mbar_wait(&full[s_now], par_now, err);
                            if (!ok) continue;
                            uint8_t* kp = ring + s_now * S::SLOT;
                            uint8_t* vp = kp + PAGE_BYTES;
                            const int tile = tf_ + j + i;
                            const int base = tile * KT;
                            if (mine && tile == t_last) {
                                // the page came from the cache as it was before this step: the new key and value go in here
                                store_vec<bf16, FE>(reinterpret_cast<bf16*>(kp + swz(new_row, lane * FE)), new_k);
                                store_vec<bf16, FE>(reinterpret_cast<bf16*>(vp + swz(new_row, lane * FE)), new_v);
                                __syncwarp();
                            }
                            if (base + KT - 1 > pos) {
                                for (int x = lane; x < 16 * NBLK * 8; x += 32) {
                                    const int r = w4 * 16 + x / (NBLK * 8), rest = x % (NBLK * 8);
                                    if (base + r > pos)
                                        *reinterpret_cast<uint4*>(vp + (rest / 8) * BLK_BYTES + r * 128 + (rest % 8) * 16) = make_uint4(0, 0, 0, 0);
                                }
                                __syncwarp();
                            }
                            float sc[2][4];
                            scores_swz<2>(sc, Qs, smem_u32(kp), w4 * 16, lane);
                            softmax_step<2>(sc, o, m, l, ph.c, row_pos, row_ok, base + w4 * 16, ph.window, lane);
                            weighted_values_swz<2>(o, sc, smem_u32(vp), w4 * 16, lane);
                            __syncwarp();
                            if (lane == 0) mbar_arrive(&empty[s_now]);
                        }
                        // ---- the four warps' results into one partial result of this run
                        constexpr int RS = HD + 2;
#pragma unroll
                        for (int r = 0; r < 2; ++r) {
                            float* dst = red + ((w4 * 16) + (lane >> 2) + r * 8) * RS;
#pragma unroll
                            for (int dt = 0; dt < DTILES; ++dt) {
                                dst[dt * 8 + (lane & 3) * 2] = o[dt][2 * r];
                                dst[dt * 8 + (lane & 3) * 2 + 1] = o[dt][2 * r + 1];
                            }
                            if ((lane & 3) == 0) { dst[HD] = m[r]; dst[HD + 1] = l[r]; }
                        }
                        named_sync(1, 128);
                        const long long seg = (long long)c + (long long)seq * ph.nkv + kvh;
                        for (int x = wt; x < Gq * HD; x += 128) {
                            const int g = x / HD, d = x % HD;
                            float mm = -INFINITY;
#pragma unroll
                            for (int w = 0; w < 4; ++w) mm = fmaxf(mm, red[(w * 16 + g) * RS + HD]);
                            float acc = 0.f, ll = 0.f;
#pragma unroll
                            for (int w = 0; w < 4; ++w) {
                                const float mw = red[(w * 16 + g) * RS + HD];
                                const float fw = mw == -INFINITY ? 0.f : exp2f(mw - mm);
                                acc += fw * red[(w * 16 + g) * RS + d];
                                ll += fw * red[(w * 16 + g) * RS + HD + 1];
                            }
                            ph.part_o[(seg * 16 + g) * HD + d] = acc;
                            if (d == 0) { ph.part_ml[(seg * 16 + g) * 2] = mm; ph.part_ml[(seg * 16 + g) * 2 + 1] = ll; }
                        }
                        named_sync(1, 128);                               // red and q are free for the next run
                        u = run_end;
                    }
                }
                n_used += (int)(u1 - u0);
            } else if (worker) {
                if (ph.type == PH_NORM) {
                    // rows dealt to the first T CTAs; every CTA clears its share of the scratch matrix
                    if (ph.zero) {
                        const long long z0 = deal_begin(ph.zero_n / 4, c, G), z1 = deal_begin(ph.zero_n / 4, c + 1, G);
                        float4* zp = reinterpret_cast<float4*>(ph.zero);
                        for (long long i = z0 + wt; i < z1; i += 128) zp[i] = make_float4(0.f, 0.f, 0.f, 0.f);
                    }
                    for (int row = c; row < T; row += G) {
                        const float* xr = sp.x + (long long)row * ph.width;
                        float ss = 0.f;
                        for (int i = wt * 4; i < ph.width; i += 512) {
                            const float4 v = __ldcg(reinterpret_cast<const float4*>(xr + i));
                            ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
                        }
                        ss = warp_sum(ss);
                        if (lane == 0) scratch[warp - 2] = ss;
                        named_sync(1, 128);
                        const float inv = inv_rms(scratch[0] + scratch[1] + scratch[2] + scratch[3], (float)ph.width, ph.eps);
                        for (int i = wt * 4; i < ph.width; i += 512) {
                            const float4 v = __ldcg(reinterpret_cast<const float4*>(xr + i));
                            const float4 g4 = *reinterpret_cast<const float4*>(ph.w + i);
                            const float ov[4] = {v.x * g4.x * inv, v.y * g4.y * inv, v.z * g4.z * inv, v.w * g4.w * inv};
                            store_vec<bf16, 4>(ph.h + (long long)row * ph.width + i, ov);
                        }
                        named_sync(1, 128);
                    }
                } else if (ph.type == PH_SILU) {
                    // pairs of neighbouring features of all tokens, dealt out over all workers of all CTAs
                    const long long n_pairs = (long long)T * ph.F / 2;
                    const long long p0 = deal_begin(n_pairs, c, G), p1 = deal_begin(n_pairs, c + 1, G);
                    for (long long i = p0 + wt; i < p1; i += 128) {
                        const long long e = i * 2;
                        const int t = (int)(e / ph.F), fcol = (int)(e % ph.F);
                        const float* row = ph.gu + (long long)t * 2 * ph.F + (fcol / 64) * 128 + (fcol % 64);
                        const float2 g2 = __ldcg(reinterpret_cast<const float2*>(row));
                        const float2 u2 = __ldcg(reinterpret_cast<const float2*>(row + 64));
                        const float ov[2] = {g2.x / (1.0f + __expf(-g2.x)) * u2.x, g2.y / (1.0f + __expf(-g2.y)) * u2.y};
                        store_vec<bf16, 2>(ph.act + (long long)t * ph.F + fcol, ov);
                    }
                } else if (ph.type == PH_MERGE) {
                    // one warp a (sequence, head): its kv head's segments merged
                    const int which = table_of(ph.window);
                    const int Gq = ph.nh / ph.nkv;
                    const long long U = attn_units(st, which, T, ph.nkv);
                    const long long items = (long long)T * ph.nh;
                    for (long long it = (long long)c * 4 + (warp - 2); it < items; it += (long long)G * 4) {
                        const int seq = (int)(it / ph.nh), head = (int)(it % ph.nh);
                        const int kvh = head / Gq, g = head % Gq;
                        const int np_ = st.np[which * MAX_SEQS + seq];
                        const long long g0 = (long long)st.cum[which * (MAX_SEQS + 1) + seq] * ph.nkv + (long long)kvh * np_;
                        const int c_first = deal_owner(g0, U, G), c_last = deal_owner(g0 + np_ - 1, U, G);
                        const long long item_kv = (long long)seq * ph.nkv + kvh;
                        // (with fewer units than CTAs some CTAs between the first and the last have no unit and
                        // wrote no segment: only CTAs with a share are read)
                        float mm = -INFINITY;
                        for (int cc = c_first; cc <= c_last; ++cc)
                            if (deal_begin(U, cc, G) < deal_begin(U, cc + 1, G)) mm = fmaxf(mm, __ldcg(ph.part_ml + ((cc + item_kv) * 16 + g) * 2));
                        float acc[FE];
#pragma unroll
                        for (int i = 0; i < FE; ++i) acc[i] = 0.f;
                        float ll = 0.f;
                        for (int cc = c_first; cc <= c_last; ++cc) {
                            if (deal_begin(U, cc, G) >= deal_begin(U, cc + 1, G)) continue;
                            const long long sg = (cc + item_kv) * 16 + g;
                            const float ms = __ldcg(ph.part_ml + sg * 2);
                            const float fs = ms == -INFINITY ? 0.f : exp2f(ms - mm);
                            ll += fs * __ldcg(ph.part_ml + sg * 2 + 1);
#pragma unroll
                            for (int i = 0; i < FE; ++i) acc[i] += fs * __ldcg(ph.part_o + sg * HD + lane * FE + i);
                        }
                        const float inv = 1.0f / ll;
#pragma unroll
                        for (int i = 0; i < FE; ++i) acc[i] *= inv;
                        store_vec<bf16, FE>(ph.o + (long long)seq * ph.nh * HD + (long long)head * HD + lane * FE, acc);
                    }
                }
            }
            // ---- the phase is done in this CTA: its stores and reductions before the count
            __threadfence();
            __syncwarp();
            named_sync(2, 160);
            if (warp == 1 && lane == 0) {
                __threadfence();
                atomicAdd(sp.counter, 1u);
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (sp.trace && c == 0 && threadIdx.x == 0) sp.trace[sp.n_phases] = global_ns();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
    if (threadIdx.x == 0 && *err) atomicExch(sp.error, 1);
}

// ---------------------------------------------------------------------------------------
UB_API int ub_stack_head_dim() { return HD; }
UB_API int ub_stack_phase_bytes() { return (int)sizeof(Phase); }
UB_API int ub_stack_slots(int bn) { return bn == 16 ? SK<16>::SLOTS : bn == 32 ? SK<32>::SLOTS : bn == 64 ? SK<64>::SLOTS : -1; }

// tensor map of a row-major bfloat16 matrix [rows, cols] (row stride ld elements): boxes of box_rows x 64 columns
UB_API int ub_stack_map_2d(void* out_map, const void* base, long long rows, long long cols, long long ld, int box_rows) {
    EncodeTiledFn enc = tensor_map_encoder();
    if (!enc) return UB_ERR_UNSUPPORTED;
    if (((uintptr_t)base & 15) || (ld * 2) % 16 != 0 || box_rows < 1 || box_rows > 256 || rows < 1 || cols < 1) return UB_ERR_ARG;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)64, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc((CUtensorMap*)out_map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (void*)base, dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : UB_ERR_ARG;
}

template <int BN>
static int launch_stack(const StackParams& sp, const MapPack& maps, int n_ctas, cudaStream_t st) {
    using S = SK<BN>;
    static bool attr_done = false;
    auto kern = decode_stack_kernel<BN>;
    if (!attr_done) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
        if (e != cudaSuccess) return (int)e;
        int per_sm = 0;
        e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, SK_THREADS, S::TOTAL);
        if (e != cudaSuccess) return (int)e;
        if (per_sm < 1) return UB_ERR_UNSUPPORTED;
        attr_done = true;
    }
    kern<<<dim3(n_ctas), dim3(SK_THREADS), S::TOTAL, st>>>(sp, maps);
    UB_LAUNCH_CHECK();
    return 0;
}

UB_API int ub_stack_max_maps() { return MAX_MAPS; }

// phases: device array of n_phases Phase records; maps: HOST array of n_maps tensor maps (128 bytes each), copied
// into the launch's parameters; counter: one zeroed word.  n_ctas must not exceed the CTAs the device holds at
// once (one an SM).
UB_API int ub_decode_stack(const void* phases, int n_phases, const void* maps, int n_maps, int T, int bn, float* x, const int* seq_before,
                           const int* table0, const int* table1, const int* table2, const int* table3, int window_b,
                           unsigned int* counter, int* error, int n_ctas, long long* trace, cudaStream_t st) {
    if (n_phases <= 0 || T <= 0) return 0;
    if (T > MAX_SEQS || T > bn || n_ctas < 1 || n_maps < 1 || n_maps > MAX_MAPS) return UB_ERR_ARG;
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (n_ctas > sms) return UB_ERR_ARG;                   // every CTA must be resident: they wait for one another
    StackParams sp;
    sp.phases = (const Phase*)phases; sp.n_phases = n_phases; sp.T = T; sp.x = x;
    static MapPack pack;                                   // (launches are made from one host thread)
    memcpy(pack.m, maps, (size_t)n_maps * sizeof(CUtensorMap));
    sp.seq_before = seq_before; sp.tables[0] = table0; sp.tables[1] = table1; sp.tables[2] = table2; sp.tables[3] = table3;
    sp.window_b = window_b; sp.counter = counter; sp.error = error; sp.trace = trace;
    switch (bn) {
        case 16: return launch_stack<16>(sp, pack, n_ctas, st);
        case 32: return launch_stack<32>(sp, pack, n_ctas, st);
        case 64: return launch_stack<64>(sp, pack, n_ctas, st);
    }
    return UB_ERR_ARG;
}
