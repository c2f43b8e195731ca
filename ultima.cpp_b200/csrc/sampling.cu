// Choosing the next token of every sequence of a batch from float32 logits, one block a row.
//
// The steps and their order are the reference sampler's (src/sampler/sampler.cpp:230-277):
// logit bias (:28-36), repetition penalty over the last repeat_last_n tokens (:41-54),
// count-based DRY penalty over the last dry_last_n (:65-83), frequency and presence
// penalties over the longer of the two windows (:86-99), temperature (<= 0: first maximum,
// :220-228, :261-263; else logits / T, :101-106), top-k (:109-121), top-p (:146-164), min-p
// (:167-176), softmax and one draw (:178-182).
//
// Two rules are this library's own.  Cuts are made by value, found by a bit-wise search
// instead of a sort, so elements equal to the cut value are all kept (the reference keeps an
// arbitrary k of them).  The draw is the inverse CDF in index order at u = hash(seed, counter),
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

// Occurrences of recent[i] inside [start, end), or 0 when an earlier index holds the same id.
__device__ __forceinline__ int count_if_first(const int* recent, int start, int end, int i) {
    const int id = recent[i];
    for (int j = start; j < i; ++j) if (recent[j] == id) return 0;
    int n = 1;
    for (int j = i + 1; j < end; ++j) n += recent[j] == id;
    return n;
}

constexpr int ST = 1024;

__global__ void __launch_bounds__(ST)
sample_kernel(const float* __restrict__ logits, long long ld, float* __restrict__ work, int V,
              const SampleParams* __restrict__ params, const int* __restrict__ recent_all,
              const int* __restrict__ bias_ids, const float* __restrict__ bias_vals,
              int* __restrict__ out_ids, unsigned long long counter_add) {
    __shared__ float red[33];
    __shared__ float seg[ST];
    __shared__ int best_idx_s[32];
    __shared__ float best_val_s[32];
    const int row = blockIdx.x, tid = threadIdx.x;
    const SampleParams p = params[row];
    const float* src = logits + (long long)row * ld;
    float* w = work + (long long)row * V;
    const bool greedy = !(p.temperature > 0.f);
    const bool plain = p.n_bias == 0 && p.n_recent == 0;
    const float* x = src;
    if (!(greedy && plain)) {
        for (int i = tid; i < V; i += ST) w[i] = src[i];
        __syncthreads();
        // 1. bias
        for (int i = tid; i < p.n_bias; i += ST) {
            const int id = bias_ids[p.bias_offset + i];
            if (id >= 0 && id < V) atomicAdd(&w[id], bias_vals[p.bias_offset + i]);
        }
        __syncthreads();
        const int* recent = recent_all + p.recent_offset;
        const int nr = p.n_recent;
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
                        w[id] -= p.dry_multiplier * powf(p.dry_base, (float)(n - p.dry_allowed_len));
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
    for (int i = tid; i < V; i += ST) {
        const float v = x[i];
        if (v > bv) { bv = v; bi = i; }            // strided: a thread's first hit is its lowest index
    }
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
    if (greedy) { if (tid == 0) out_ids[row] = imax == 0x7fffffff ? 0 : imax; return; }

    // 5. temperature (in place); from here on the maximum is vmax / T
    const float invT = 1.0f / p.temperature;
    if (p.temperature != 1.0f) {
        for (int i = tid; i < V; i += ST) w[i] *= invT;
        __syncthreads();
    }
    const float m = p.temperature != 1.0f ? vmax * invT : vmax;
    unsigned cut = 0;                             // keep keys >= cut
    // 6. top-k: the largest cut that still keeps k elements
    if (p.top_k > 0 && p.top_k < V) {
        unsigned t = 0;
        for (int bit = 31; bit >= 0; --bit) {
            const unsigned cand = t | (1u << bit);
            float cnt = 0.f;
            for (int i = tid; i < V; i += ST) cnt += key_of(w[i]) >= cand ? 1.f : 0.f;
            cnt = block_sum(cnt, red);
            if (cnt >= (float)p.top_k) t = cand;
        }
        cut = t;
    }
    // 7. top-p: the largest cut whose kept mass reaches p of the mass kept so far
    if (p.top_p < 1.0f && p.top_p > 0.f) {
        float z = 0.f;
        for (int i = tid; i < V; i += ST) z += key_of(w[i]) >= cut ? expf(w[i] - m) : 0.f;
        z = block_sum(z, red);
        const float need = p.top_p * z;
        unsigned t = cut;
        for (int bit = 31; bit >= 0; --bit) {
            if (t & (1u << bit)) continue;
            const unsigned cand = t | (1u << bit);
            float mass = 0.f;
            for (int i = tid; i < V; i += ST) mass += key_of(w[i]) >= cand ? expf(w[i] - m) : 0.f;
            mass = block_sum(mass, red);
            if (mass >= need) t = cand;
        }
        cut = t;
    }
    // 8. min-p: drop p_i < min_p * p_max, i.e. exp(x_i - m) < min_p
    const float minp = p.min_p > 0.f ? p.min_p : 0.f;
    // 9. draw: inverse CDF in index order; thread t owns one contiguous stretch
    const int per = (V + ST - 1) / ST;
    const int b = tid * per, e = min(V, b + per);
    float local = 0.f;
    for (int i = b; i < e; ++i) {
        const float v = w[i];
        const float pe = expf(v - m);
        local += (key_of(v) >= cut && pe >= minp) ? pe : 0.f;
    }
    seg[tid] = local;
    __syncthreads();
    if (tid == 0) {                               // exclusive prefix, in order
        float run = 0.f;
        for (int i = 0; i < ST; ++i) { const float s = seg[i]; seg[i] = run; run += s; }
        red[0] = run;
        const unsigned long long r = mix64s(p.seed ^ mix64s(p.counter + counter_add + 0x632BE59BD9B4E019ull));
        red[1] = (float)(unsigned)(r >> 40) * (1.0f / 16777216.0f);
        best_idx_s[1] = imax;                     // fallback: the maximum
    }
    __syncthreads();
    const float total = red[0];
    const float target = red[1] * total;
    const float before = seg[tid];
    const float after = tid + 1 < ST ? seg[tid + 1] : total;
    // the owner of the target: before <= target < after (the last non-empty stretch takes the end)
    if (e > b && target >= before && (target < after)) {
        float run = before;
        int pick = -1;
        for (int i = b; i < e; ++i) {
            const float v = w[i];
            const float pe = expf(v - m);
            const float pr = (key_of(v) >= cut && pe >= minp) ? pe : 0.f;
            if (pr > 0.f) { run += pr; if (target < run) { pick = i; break; } pick = i; }
        }
        if (pick >= 0) best_idx_s[1] = pick;
    }
    __syncthreads();
    if (tid == 0) out_ids[row] = best_idx_s[1];
}

// ``counter_add`` is added to every row's counter (a batch whose rows have drawn equally often can
// keep its records on the device and pass the count here).
UB_API int ub_sample(const float* logits, long long ld, float* work, int n_rows, int V,
                     const void* params, const int* recent, const int* bias_ids, const float* bias_vals,
                     int* out_ids, unsigned long long counter_add, cudaStream_t st) {
    if (n_rows <= 0) return 0;
    if (V <= 0) return UB_ERR_ARG;
    sample_kernel<<<n_rows, ST, 0, st>>>(logits, ld, work, V, (const SampleParams*)params, recent,
                                         bias_ids, bias_vals, out_ids, counter_add);
    UB_LAUNCH_CHECK();
    return 0;
}
UB_API int ub_sample_params_size() { return (int)sizeof(SampleParams); }
