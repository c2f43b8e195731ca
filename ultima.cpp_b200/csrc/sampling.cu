// Choosing the next token of every sequence of a batch from float32 logits, one block a row.
//
// The steps and their order are the reference sampler's (src/sampler/sampler.cpp:230-277):
// logit bias (:28-36), repetition penalty over the last repeat_last_n tokens (:41-54),
// count-based DRY penalty over the last dry_last_n (:65-83), frequency and presence
// penalties over the longer of the two windows (:86-99), temperature (<= 0: first maximum,
// :220-228, :261-263; else logits / T, :101-106), top-k (:109-121), top-p (:146-164), min-p
// (:167-176), softmax and one draw (:178-182).
//
// Two rules are this library's own.  Cuts are made by value, found by bucket histograms
// instead of a sort (see "Where to cut" below), so elements equal to the cut value are all kept
// (the reference keeps an arbitrary k of them).  The draw is the inverse CDF in index order at u = hash(seed, counter),
// one stream for each sequence, so a sequence's tokens do not depend on its batch (the
// reference draws from a std::mt19937_64 it owns for one sequence).
#include "common.cuh"

struct SampleParams {
    float temperature, top_p, min_p, rep_penalty;
    float freq_penalty, presence_penalty, dry_multiplier, dry_base;
    int top_k, repeat_last_n, dry_last_n, dry_allowed_len;
    int n_recent, recent_offset, n_bias, bias_offset;
    unsigned long long seed, counter;
};

__device__ __forceinline__ unsigned key_of(float x) {
    const unsigned b = __float_as_uint(x);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ unsigned long long mix64s(unsigned long long z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

// The recent tokens of a row, oldest first: a stretch of a flat array that the host sent with the
// call, or the last tokens of a ring that stays on the device and that the kernel itself appends
// each sampled token to (cap > 0: element j lies at (first + j) mod cap).
struct Window {
    const int* base;
    int first, cap;
    __device__ __forceinline__ int operator[](int j) const {
        const int k = first + j;
        return base[cap > 0 ? k % cap : k];
    }
};

// Occurrences of recent[i] inside [start, end), or 0 when an earlier index holds the same id.
// One loop without branches: every thread of a warp reads the same element at the same time.
__device__ __forceinline__ int count_if_first(const Window& recent, int start, int end, int i) {
    const int id = recent[i];
    int n = 0, earlier = 0;
    if (recent.cap == 0) {
        const int* r = recent.base + recent.first;
#pragma unroll 8
        for (int j = start; j < end; ++j) {
            const int same = r[j] == id;
            n += same;
            earlier |= same & (j < i);
        }
    } else {
        for (int j = start; j < end; ++j) {
            const int same = recent[j] == id;
            n += same;
            earlier |= same & (j < i);
        }
    }
    return earlier ? 0 : n;
}

constexpr int ST = 1024;
constexpr int WIN_SMEM = 1024;            // recent tokens of a row that are held in shared memory

// Every element of x[0, V) once, as f(index, value): four neighbouring elements a load where the
// row allows it, several loads in flight.  A thread meets its indices in rising order.
template <typename F>
__device__ __forceinline__ void visit(const float* x, int V, int tid, F f) {
    const int head = min(V, (int)(((16u - (unsigned)((uintptr_t)x & 15u)) & 15u) >> 2));
    if (tid < head) f(tid, x[tid]);
    const float4* x4 = reinterpret_cast<const float4*>(x + head);
    const int n4 = (V - head) >> 2;
#pragma unroll 4
    for (int i = tid; i < n4; i += ST) {
        const float4 v = x4[i];
        const int b = head + 4 * i;
        f(b, v.x); f(b + 1, v.y); f(b + 2, v.z); f(b + 3, v.w);
    }
    const int t = head + 4 * n4 + tid;
    if (t < V) f(t, x[t]);
}

// ---------------------------------------------------------------------------------------
// Where to cut: the largest key t such that the kept elements with key >= t weigh at least
// ``need`` (weight 1 each for top-k, exp(x - max) for top-p, the latter as a 64-bit fixed-point
// integer so that a sum does not depend on the order of its terms).  Instead of 32 passes over
// the row (one a bit of the key) it takes three: a histogram of 1024 buckets over the 64 logit
// units below the maximum, a histogram of 1024 parts of the bucket that holds the cut, then the
// elements of that part (a handful) are copied to shared memory and ranked there.  The histograms
// only say where to look (counts are exact; masses are float sums in arrival order); the pass that
// copies the elements also sums, exactly, what lies above them, and the ranking is exact.  A row
// that does not fit (the cut lies further than 64 units below the maximum, more than LIST elements
// share the last part, or the float sums pointed one part off) takes the bit-by-bit search, which
// answers the same question with the same integers, so both ways give the same cut.
// ---------------------------------------------------------------------------------------
constexpr int NB = 1024;
constexpr int LIST = 2048;
constexpr int SMALL = 512;             // survivors that the rest of the ladder handles in shared memory (ranked pair by pair)
constexpr float BUCKET_SCALE = (float)NB / 64.0f;
constexpr float FIXED_ONE = 1099511627776.0f;              // 2^40
typedef unsigned long long u64;

struct SelectSmem {
    union { float f[NB]; unsigned u[NB]; } hist;
    union { float f[32]; unsigned u[32]; } warp_tot;
    u64 red64[33];
    float list_v[LIST];
    u64 list_w[LIST];
    int list_i[LIST];
    float found_above_f;
    unsigned found_above_u;
    int found_bucket, count;
    unsigned best;
};

template <bool MASS>
__device__ __forceinline__ u64 weight_of(float v, float m) {
    if (!MASS) return 1ull;
    const float d = __fsub_rn(v, m);
    return d < -28.0f ? 0ull : (u64)__fmul_rn(expf(d), FIXED_ONE);       // below that the product is under one anyway
}
// bucket (0: at the maximum) and part of the bucket of a value; both fall as the value rises
__device__ __forceinline__ void place_of(float v, float m, int& bucket, int& part) {
    // single operations, never fused with what comes before: every pass must place a value alike
    const float d = __fmul_rn(__fsub_rn(m, v), BUCKET_SCALE);
    if (!(d < (float)(NB - 1))) { bucket = NB - 1; part = NB - 1; return; }
    bucket = d > 0.f ? (int)d : 0;
    const float f = __fmul_rn(__fsub_rn(d, (float)bucket), (float)NB);
    part = f > 0.f ? min(NB - 1, (int)f) : 0;
}

__device__ __forceinline__ u64 block_sum_u64(u64 v, u64* red, int tid) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if ((tid & 31) == 0) red[tid >> 5] = v;
    __syncthreads();
    if (tid == 0) {
        u64 t = 0;
        for (int w = 0; w < ST / 32; ++w) t += red[w];
        red[32] = t;
    }
    __syncthreads();
    return red[32];
}

__device__ __forceinline__ void note_above(SelectSmem& sm, float v) { sm.found_above_f = v; }
__device__ __forceinline__ void note_above(SelectSmem& sm, unsigned v) { sm.found_above_u = v; }

// The first bucket b with hist[0] + ... + hist[b] >= need (thread b holds hist[b]); its index and
// the sum before it go to shared memory.  found_bucket stays -1 when the whole sum is too small.
template <typename T>
__device__ __forceinline__ void first_reaching(SelectSmem& sm, T* hist, T* warp_tot, T need, int tid) {
    const int lane = tid & 31, warp = tid >> 5;
    const T own = hist[tid];
    T incl = own;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const T up = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += up;
    }
    if (lane == 31) warp_tot[warp] = incl;
    if (tid == 0) sm.found_bucket = -1;
    __syncthreads();
    T before = 0;
    for (int w = 0; w < warp; ++w) before += warp_tot[w];
    incl += before;
    if (incl >= need && incl - own < need) {
        sm.found_bucket = tid;
        note_above(sm, (T)(incl - own));
    }
    __syncthreads();
}

template <bool MASS>
__device__ bool select_in_bucket(const float* x, float sc, int V, float m, unsigned old_cut, u64 need, SelectSmem& sm,
                                 int tid, int b1, float above1_f, unsigned above1_u, unsigned& cut_out);

template <bool MASS>
__device__ bool select_cut(const float* x, float sc, int V, float m, unsigned old_cut, u64 need, SelectSmem& sm,
                           int tid, unsigned& cut_out) {
    static_assert(NB == ST, "one thread a bucket");
    // buckets (what lies further than the last bucket below the maximum is not counted: a cut that far
    // down is not found here)
    sm.hist.u[tid] = 0;
    __syncthreads();
    visit(x, V, tid, [&](int, float raw) {
        const float v = __fmul_rn(raw, sc);
        if (key_of(v) < old_cut) return;
        int b, part;
        place_of(v, m, b, part);
        if (b < NB - 1) {
            if (MASS) atomicAdd(&sm.hist.f[b], expf(__fsub_rn(v, m)));
            else atomicAdd(&sm.hist.u[b], 1u);
        }
    });
    __syncthreads();
    const float need_f = (float)need * (1.0f / FIXED_ONE);
    if (MASS) first_reaching<float>(sm, sm.hist.f, sm.warp_tot.f, need_f, tid);
    else first_reaching<unsigned>(sm, sm.hist.u, sm.warp_tot.u, (unsigned)need, tid);
    const int b1 = sm.found_bucket;
    if (b1 < 0) return false;
    return select_in_bucket<MASS>(x, sc, V, m, old_cut, need, sm, tid, b1, sm.found_above_f, sm.found_above_u, cut_out);
}

// The second and third pass of the above, given the bucket b1 that holds the cut and what the
// histogram summed before it.
template <bool MASS>
__device__ bool select_in_bucket(const float* x, float sc, int V, float m, unsigned old_cut, u64 need, SelectSmem& sm,
                                 int tid, int b1, float above1_f, unsigned above1_u, unsigned& cut_out) {
    const float need_f = (float)need * (1.0f / FIXED_ONE);
    // parts of that bucket
    __syncthreads();
    sm.hist.u[tid] = 0;
    __syncthreads();
    visit(x, V, tid, [&](int, float raw) {
        const float v = __fmul_rn(raw, sc);
        if (key_of(v) < old_cut) return;
        int b, part;
        place_of(v, m, b, part);
        if (b == b1) {
            if (MASS) atomicAdd(&sm.hist.f[part], expf(__fsub_rn(v, m)));
            else atomicAdd(&sm.hist.u[part], 1u);
        }
    });
    __syncthreads();
    if (MASS) first_reaching<float>(sm, sm.hist.f, sm.warp_tot.f, fmaxf(need_f - above1_f, 1e-30f), tid);
    else first_reaching<unsigned>(sm, sm.hist.u, sm.warp_tot.u, (unsigned)need - above1_u, tid);
    const int b2 = sm.found_bucket;
    if (b2 < 0) return false;
    // the elements of that part, and the exact weight of everything above it
    if (tid == 0) { sm.count = 0; sm.best = 0; }
    __syncthreads();
    u64 above_l = 0;
    visit(x, V, tid, [&](int, float raw) {
        const float v = __fmul_rn(raw, sc);
        if (key_of(v) < old_cut) return;
        int b, part;
        place_of(v, m, b, part);
        if (b < b1 || (b == b1 && part < b2)) above_l += weight_of<MASS>(v, m);
        else if (b == b1 && part == b2) {
            const int at = atomicAdd(&sm.count, 1);
            if (at < LIST) { sm.list_v[at] = v; sm.list_w[at] = weight_of<MASS>(v, m); }
        }
    });
    const u64 above = block_sum_u64(above_l, sm.red64, tid);
    const int n = sm.count;
    if (n > LIST || above >= need) return false;
    // the element with the largest key whose own weight and that of all larger ones reach the need
    const u64 left = need - above;
    for (int e = tid; e < n; e += ST) {
        const unsigned ke = key_of(sm.list_v[e]);
        u64 sum = 0;
        for (int j = 0; j < n; ++j) sum += key_of(sm.list_v[j]) >= ke ? sm.list_w[j] : 0ull;
        if (sum >= left) atomicMax(&sm.best, ke);
    }
    __syncthreads();
    cut_out = sm.best;
    return sm.best != 0;
}

// The same cut, one bit of the key a pass over the row.
template <bool MASS>
__device__ unsigned search_cut(const float* x, float sc, int V, float m, unsigned old_cut, u64 need, SelectSmem& sm,
                               int tid) {
    unsigned t = 0;
    for (int bit = 31; bit >= 0; --bit) {
        const unsigned cand = t | (1u << bit);
        u64 sum = 0;
        visit(x, V, tid, [&](int, float raw) {
            const float v = __fmul_rn(raw, sc);
            const unsigned k = key_of(v);
            if (k >= cand && k >= old_cut) sum += weight_of<MASS>(v, m);
        });
        if (block_sum_u64(sum, sm.red64, tid) >= need) t = cand;
    }
    return t;
}

// top-k in two passes when what lies at and above the cut's bucket is a handful: the count histogram
// as above, then every element of those buckets (value and index) is copied to shared memory, where the
// cut is the k-th largest of them.  The copied elements are what the rest of the ladder works on.
// False (nothing changed that matters) when the bucket is not found or holds too much.
__device__ bool topk_collect(const float* x, float sc, int V, float m, int k, SelectSmem& sm, int tid,
                             unsigned& cut_out, int& n_out) {
    sm.hist.u[tid] = 0;
    __syncthreads();
    visit(x, V, tid, [&](int, float raw) {
        const float v = __fmul_rn(raw, sc);
        int b, part;
        place_of(v, m, b, part);
        if (b < NB - 1) atomicAdd(&sm.hist.u[b], 1u);
    });
    __syncthreads();
    first_reaching<unsigned>(sm, sm.hist.u, sm.warp_tot.u, (unsigned)k, tid);
    const int b1 = sm.found_bucket;
    if (b1 < 0) return false;
    const unsigned expect = sm.found_above_u + sm.hist.u[b1];
    if (expect > (unsigned)SMALL) return false;
    if (tid == 0) { sm.count = 0; sm.best = 0; }
    __syncthreads();
    visit(x, V, tid, [&](int i, float raw) {
        const float v = __fmul_rn(raw, sc);
        int b, part;
        place_of(v, m, b, part);
        if (b <= b1) {
            const int at = atomicAdd(&sm.count, 1);
            if (at < LIST) { sm.list_v[at] = v; sm.list_i[at] = i; }
        }
    });
    __syncthreads();
    const int n = sm.count;
    if (n > SMALL || n < k) return false;
    for (int e = tid; e < n; e += ST) {
        const unsigned ke = key_of(sm.list_v[e]);
        int c = 0;
        for (int j = 0; j < n; ++j) c += key_of(sm.list_v[j]) >= ke;
        if (c >= k) atomicMax(&sm.best, ke);
    }
    __syncthreads();
    cut_out = sm.best;
    n_out = n;
    return sm.best != 0;
}

// top-p, first pass: the kept elements' total mass (exact) and the histogram of masses in one go, then
// the bucket b1 where the mass reaches the need.  If the buckets down to b1 + 1 (one more for the
// float sums' sake) hold little enough (a peaked distribution; counted in a pass of its own, no
// atomics), their elements are copied to shared memory and n_out says how many: the caller finds
// the cut among them with exact sums and checks that it is there.  Else n_out is -1 and the caller
// goes on from b1 with the passes over the row.
__device__ void topp_first(const float* x, float sc, int V, float m, unsigned old_cut, float top_p, SelectSmem& sm,
                           int tid, u64& z_out, u64& need_out, int& b1_out, int& n_out) {
    sm.hist.f[tid] = 0.f;
    __syncthreads();
    u64 zl = 0;
    visit(x, V, tid, [&](int, float raw) {
        const float v = __fmul_rn(raw, sc);
        if (key_of(v) < old_cut) return;
        zl += weight_of<true>(v, m);
        int b, part;
        place_of(v, m, b, part);
        if (b < NB - 1) atomicAdd(&sm.hist.f[b], expf(__fsub_rn(v, m)));
    });
    const u64 z = block_sum_u64(zl, sm.red64, tid);
    u64 need = (u64)((double)top_p * (double)z);
    if (need < 1) need = 1;
    first_reaching<float>(sm, sm.hist.f, sm.warp_tot.f, (float)need * (1.0f / FIXED_ONE), tid);
    z_out = z; need_out = need; b1_out = sm.found_bucket; n_out = -1;
    const int b1 = sm.found_bucket;
    if (b1 < 0 || b1 + 1 >= NB - 1) return;
    u64 mine = 0;
    visit(x, V, tid, [&](int, float raw) {
        const float v = __fmul_rn(raw, sc);
        if (key_of(v) < old_cut) return;
        int b, part;
        place_of(v, m, b, part);
        mine += b <= b1 + 1;
    });
    if (block_sum_u64(mine, sm.red64, tid) > (u64)SMALL) return;
    if (tid == 0) { sm.count = 0; sm.best = 0; }
    __syncthreads();
    visit(x, V, tid, [&](int i, float raw) {
        const float v = __fmul_rn(raw, sc);
        if (key_of(v) < old_cut) return;
        int b, part;
        place_of(v, m, b, part);
        if (b <= b1 + 1) {
            const int at = atomicAdd(&sm.count, 1);
            if (at < LIST) { sm.list_v[at] = v; sm.list_i[at] = i; }
        }
    });
    __syncthreads();
    n_out = sm.count <= SMALL ? sm.count : -1;
}

__global__ void __launch_bounds__(ST)
sample_kernel(const float* __restrict__ logits, long long ld, float* __restrict__ work, int V,
              const SampleParams* __restrict__ params, const int* __restrict__ recent_all,
              const int* __restrict__ bias_ids, const float* __restrict__ bias_vals,
              int* __restrict__ out_ids, unsigned long long counter_add, int* __restrict__ hist,
              int* __restrict__ hist_len, int hist_cap) {
    __shared__ float red[33];
    __shared__ float seg[34];
    __shared__ int best_idx_s[32];
    __shared__ float best_val_s[32];
    __shared__ SelectSmem sel;
    __shared__ int win_s[WIN_SMEM];
    const int row = blockIdx.x, tid = threadIdx.x;
    const SampleParams p = params[row];
    const float* src = logits + (long long)row * ld;
    float* w = work + (long long)row * V;
    const bool greedy = !(p.temperature > 0.f);
    const bool plain = p.n_bias == 0 && p.n_recent == 0;
    // n_recent < 0: the row's history is ring number recent_offset on the device
    const bool ring = p.n_recent < 0 && hist != nullptr && hist_cap > 0;
    const int n_total = ring ? hist_len[p.recent_offset] : 0;
    int* my_ring = ring ? hist + (long long)p.recent_offset * hist_cap : nullptr;
    const float* x = src;
    if (!plain) {
        visit(src, V, tid, [&](int i, float v) { w[i] = v; });
        __syncthreads();
        // 1. bias
        for (int i = tid; i < p.n_bias; i += ST) {
            const int id = bias_ids[p.bias_offset + i];
            if (id >= 0 && id < V) atomicAdd(&w[id], bias_vals[p.bias_offset + i]);
        }
        __syncthreads();
        const int nr = ring ? min(n_total, hist_cap) : max(p.n_recent, 0);
        Window recent = ring ? Window{my_ring, (n_total - nr) % hist_cap, hist_cap}
                             : Window{recent_all + p.recent_offset, 0, 0};
        if (nr <= WIN_SMEM) {                     // the usual case: the window is read from shared memory
            for (int j = tid; j < nr; j += ST) win_s[j] = recent[j];
            __syncthreads();
            recent = Window{win_s, 0, 0};
        }
        // 2. repetition penalty
        if (p.rep_penalty != 1.0f && p.repeat_last_n > 0 && nr > 0) {
            const int start = max(0, nr - p.repeat_last_n);
            for (int i = start + tid; i < nr; i += ST) {
                const int id = recent[i];
                if (id < 0 || id >= V) continue;
                if (count_if_first(recent, start, nr, i) > 0) {
                    const float l = w[id];
                    w[id] = l > 0.f ? l / p.rep_penalty : l * p.rep_penalty;
                }
            }
            __syncthreads();
        }
        // 3. DRY
        if (p.dry_multiplier > 0.f && p.dry_last_n > 0) {
            const int start = max(0, nr - p.dry_last_n);
            if (nr - start >= 2) {
                for (int i = start + tid; i < nr; i += ST) {
                    const int id = recent[i];
                    if (id < 0 || id >= V) continue;
                    const int n = count_if_first(recent, start, nr, i);
                    if (n > p.dry_allowed_len)
                        w[id] -= p.dry_multiplier * exp2f(log2f(p.dry_base) * (float)(n - p.dry_allowed_len));
                }
            }
            __syncthreads();
        }
        // 4. frequency / presence
        if (p.freq_penalty != 0.f || p.presence_penalty != 0.f) {
            const int win = max(p.repeat_last_n, p.dry_last_n);
            const int start = win > 0 ? max(0, nr - win) : nr;
            for (int i = start + tid; i < nr; i += ST) {
                const int id = recent[i];
                if (id < 0 || id >= V) continue;
                const int n = count_if_first(recent, start, nr, i);
                if (n > 0) { w[id] -= (float)n * p.freq_penalty; w[id] -= p.presence_penalty; }
            }
            __syncthreads();
        }
        x = w;
    }
    // maximum and its first index
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    visit(x, V, tid, [&](int i, float v) {
        if (v > bv) { bv = v; bi = i; }            // indices rise: a thread's first hit is its lowest index
    });
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if ((tid & 31) == 0) { best_val_s[tid >> 5] = bv; best_idx_s[tid >> 5] = bi; }
    __syncthreads();
    if (tid < 32) {
        bv = best_val_s[tid]; bi = best_idx_s[tid];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if (tid == 0) { best_val_s[0] = bv; best_idx_s[0] = bi; }
    }
    __syncthreads();
    const float vmax = best_val_s[0];
    const int imax = best_idx_s[0];
    if (greedy) {
        if (tid == 0) {
            const int id = imax == 0x7fffffff ? 0 : imax;
            out_ids[row] = id;
            if (ring) { my_ring[n_total % hist_cap] = id; hist_len[p.recent_offset] = n_total + 1; }
        }
        return;
    }

    // 5. temperature: every later read takes x[i] * sc; the maximum is vmax * sc
    const float sc = p.temperature != 1.0f ? 1.0f / p.temperature : 1.0f;
    const float m = vmax * sc;
    unsigned cut = 0;                             // keep keys >= cut
    // 6. top-k: the largest cut that still keeps k elements
    int n_list = -1;                              // >= 0: what top-k kept (and a few below it) lies in shared memory
    if (p.top_k > 0 && p.top_k < V) {
        unsigned t = 0;
        if (!topk_collect(x, sc, V, m, p.top_k, sel, tid, t, n_list)) {
            n_list = -1;
            __syncthreads();
            if (!select_cut<false>(x, sc, V, m, 0u, (u64)p.top_k, sel, tid, t))
                t = search_cut<false>(x, sc, V, m, 0u, (u64)p.top_k, sel, tid);
        }
        cut = t;
    }
    const float minp = p.min_p > 0.f ? p.min_p : 0.f;
    // What top-k left is usually a few dozen elements: once they are in shared memory, everything
    // that follows (top-p, min-p, the draw) happens there instead of in passes over the row.
    // top-p where top-k has left no list (it is off, or it kept too much): the first pass over the row,
    // and a list if what top-p keeps is little
    u64 z_all = 0, need_all = 0;                  // the kept elements' mass and the share of it that top-p asks for
    int b1_p = -1;
    const bool p_first = n_list < 0 && p.top_p < 1.0f && p.top_p > 0.f;
    if (p_first) topp_first(x, sc, V, m, cut, p.top_p, sel, tid, z_all, need_all, b1_p, n_list);
    __syncthreads();
    if ((cut != 0 && !p_first) || n_list >= 0) {
        if (n_list < 0) {
            if (tid == 0) { sel.count = 0; sel.best = 0; }
            __syncthreads();
            visit(x, V, tid, [&](int i, float raw) {
                const float v = __fmul_rn(raw, sc);
                if (key_of(v) < cut) return;
                const int at = atomicAdd(&sel.count, 1);
                if (at < LIST) { sel.list_v[at] = v; sel.list_i[at] = i; }
            });
            __syncthreads();
            n_list = sel.count;
        }
        const int n = n_list;
        if (n <= SMALL) {
            if (tid == 0) sel.best = 0;
            // elements below the cut (the list may hold some) weigh nothing
            for (int e = tid; e < n; e += ST)
                sel.list_w[e] = key_of(sel.list_v[e]) >= cut ? weight_of<true>(sel.list_v[e], m) : 0ull;
            __syncthreads();
            unsigned cut2 = cut;
            bool found = true;
            if (p.top_p < 1.0f && p.top_p > 0.f) {
                u64 zl = 0;
                for (int e = tid; e < n; e += ST) zl += sel.list_w[e];
                u64 zi = block_sum_u64(zl, sel.red64, tid);
                if (z_all) zi = z_all;
                u64 need_i = (u64)((double)p.top_p * (double)zi);
                if (need_i < 1) need_i = 1;
                for (int e = tid; e < n; e += ST) {
                    const unsigned ke = key_of(sel.list_v[e]);
                    u64 sum = 0;
                    for (int j = 0; j < n; ++j) sum += key_of(sel.list_v[j]) >= ke ? sel.list_w[j] : 0ull;
                    if (sum >= need_i) atomicMax(&sel.best, ke);
                }
                __syncthreads();
                if (sel.best > cut2) cut2 = sel.best;
                found = sel.best != 0;            // the cut lies in the list (always, when the list is all that is kept)
            }
            __syncthreads();
            if (found) {
            // probabilities of the survivors, then the draw in index order: element e stands at the
            // number of survivors with a smaller index
            for (int e = tid; e < n; e += ST) {
                const float v = sel.list_v[e];
                const float d = __fsub_rn(v, m);
                float pe = (key_of(v) < cut2 || d < -87.0f) ? 0.f : expf(d);
                if (pe < minp) pe = 0.f;
                int rank = 0;
                const int ie = sel.list_i[e];
                for (int j = 0; j < n; ++j) rank += sel.list_i[j] < ie;
                reinterpret_cast<float*>(sel.list_w)[rank] = pe;               // the weights are no longer needed
                reinterpret_cast<int*>(sel.list_w)[LIST + rank] = ie;
            }
            __syncthreads();
            if (tid == 0) {
                const float* pr = reinterpret_cast<const float*>(sel.list_w);
                const int* id = reinterpret_cast<const int*>(sel.list_w) + LIST;
                float total = 0.f;
                for (int j = 0; j < n; ++j) total += pr[j];
                const unsigned long long r = mix64s(p.seed ^ mix64s(p.counter + counter_add + 0x632BE59BD9B4E019ull));
                const float target = (float)(unsigned)(r >> 40) * (1.0f / 16777216.0f) * total;
                float run = 0.f;
                int pick = imax;
                for (int j = 0; j < n; ++j) {
                    if (pr[j] > 0.f) { run += pr[j]; pick = id[j]; if (target < run) break; }
                }
                out_ids[row] = pick;
                if (ring) { my_ring[n_total % hist_cap] = pick; hist_len[p.recent_offset] = n_total + 1; }
            }
            return;
            }
        }
    }
    // 7. top-p: the largest cut whose kept mass reaches p of the mass kept so far
    if (p.top_p < 1.0f && p.top_p > 0.f) {
        // the first pass has been made (topp_first): on from its bucket
        __syncthreads();
        unsigned t = cut;
        first_reaching<float>(sel, sel.hist.f, sel.warp_tot.f, (float)need_all * (1.0f / FIXED_ONE), tid);
        bool ok = b1_p >= 0 && sel.found_bucket == b1_p;
        if (ok) ok = select_in_bucket<true>(x, sc, V, m, cut, need_all, sel, tid, b1_p, sel.found_above_f, 0u, t);
        if (!ok) t = search_cut<true>(x, sc, V, m, cut, need_all, sel, tid);
        cut = t > cut ? t : cut;
    }
    // 8. min-p: drop p_i < min_p * p_max, i.e. exp(x_i - m) < min_p (minp above)
    // 9. draw: inverse CDF in index order.  Warp w owns the stretch [w * C, (w + 1) * C) and reads it
    // row by row of 32 neighbours; the warp that holds the target walks its stretch once more.
    const int lane = tid & 31, warp = tid >> 5;
    const int C = (((V + 31) / 32 + 31) / 32) * 32;           // a stretch: whole rows
    const int c0 = warp * C, c1 = min(V, c0 + C);
    auto kept = [&](int i) -> float {
        const float v = __fmul_rn(x[i], sc);
        // what was cut away, and what is too small for a float that is not denormal, needs no exp
        const float d = __fsub_rn(v, m);
        if (key_of(v) < cut || d < -87.0f) return 0.f;
        const float pe = expf(d);
        return pe >= minp ? pe : 0.f;
    };
    float local = 0.f;
#pragma unroll 4
    for (int i = c0 + lane; i < c1; i += 32) local += kept(i);
    local = warp_sum(local);
    if (lane == 0) seg[warp] = local;
    __syncthreads();
    if (tid == 0) {                               // exclusive prefix over the stretches, in order
        float run = 0.f;
        for (int i = 0; i < 32; ++i) { const float t = seg[i]; seg[i] = run; run += t; }
        seg[32] = run;
        const unsigned long long r = mix64s(p.seed ^ mix64s(p.counter + counter_add + 0x632BE59BD9B4E019ull));
        red[1] = (float)(unsigned)(r >> 40) * (1.0f / 16777216.0f);
        best_idx_s[1] = imax;                     // fallback: the maximum
    }
    __syncthreads();
    const float total = seg[32];
    const float target = red[1] * total;
    const float before = seg[warp];
    const float after = seg[warp + 1];
    // the owner of the target: before <= target < after (rounding may leave the very end to nobody:
    // the maximum stands in)
    if (c1 > c0 && target >= before && target < after) {
        float run = before;
        int pick = -1;
        for (int r0 = c0; r0 < c1; r0 += 32) {
            const int i = r0 + lane;
            const float pr = i < c1 ? kept(i) : 0.f;
            float incl = pr;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const float up = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += up;
            }
            const unsigned has = __ballot_sync(0xffffffffu, pr > 0.f);
            const unsigned hit = __ballot_sync(0xffffffffu, pr > 0.f && target < run + incl);
            if (hit) { pick = r0 + __ffs(hit) - 1; break; }
            if (has) pick = r0 + 31 - __clz(has);          // the last kept element so far
            run += __shfl_sync(0xffffffffu, incl, 31);
        }
        if (lane == 0 && pick >= 0) best_idx_s[1] = pick;
    }
    __syncthreads();
    if (tid == 0) {
        const int id = best_idx_s[1];
        out_ids[row] = id;
        if (ring) { my_ring[n_total % hist_cap] = id; hist_len[p.recent_offset] = n_total + 1; }
    }
}

// ``counter_add`` is added to every row's counter (a batch whose rows have drawn equally often can
// keep its records on the device and pass the count here).  A row whose record has n_recent < 0
// takes its recent tokens from ring number recent_offset of ``hist`` ([rings, hist_cap] int32, with
// ``hist_len`` tokens put into it so far) and appends the token it samples.
UB_API int ub_sample(const float* logits, long long ld, float* work, int n_rows, int V,
                     const void* params, const int* recent, const int* bias_ids, const float* bias_vals,
                     int* out_ids, unsigned long long counter_add, int* hist, int* hist_len, int hist_cap,
                     cudaStream_t st) {
    if (n_rows <= 0) return 0;
    if (V <= 0 || hist_cap < 0 || (hist_cap > 0 && (!hist || !hist_len))) return UB_ERR_ARG;
    sample_kernel<<<n_rows, ST, 0, st>>>(logits, ld, work, V, (const SampleParams*)params, recent,
                                         bias_ids, bias_vals, out_ids, counter_add, hist, hist_len, hist_cap);
    UB_LAUNCH_CHECK();
    return 0;
}
UB_API int ub_sample_params_size() { return (int)sizeof(SampleParams); }

