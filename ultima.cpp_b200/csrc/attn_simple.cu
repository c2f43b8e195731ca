// Attention over the paged cache, one block for each (query token, query head), any head size
// up to 256, float32 or bfloat16 storage, float32 arithmetic throughout.
//
// It restates the reference's per-token loop (src/model/qwen_block.cpp:94-135): scores
// q.k * scale over the visible positions, max-shifted softmax (src/kernels/softmax.cpp:9-29),
// weighted sum of the values; query head h reads KV head h / (nh / nkv); a token at position
// p sees positions (p - window, p] (src/model/qwen_block.cpp:742-745).  Keys are taken in
// chunks with a running maximum, so the context length is not bounded by shared memory.
// The order of every sum depends only on the key range, never on the batch.
#include "common.cuh"

constexpr int CHUNK = 512;

template <typename TQ, typename TC>
__global__ void __launch_bounds__(128)
attn_simple_kernel(const TQ* __restrict__ q, long long q_stride, const TC* __restrict__ kc,
                   const TC* __restrict__ vc, TQ* __restrict__ out, long long o_stride,
                   const int* __restrict__ tok_pos, const int* __restrict__ tok_seq, PagedKV c,
                   int nh, int window, float scale) {
    extern __shared__ float smem[];
    float* qs = smem;                    // [hd]
    float* sc = smem + c.head_dim;       // [CHUNK]
    __shared__ float red[33];
    const int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
    const int hd = c.head_dim;
    const int kvh = h / (nh / c.n_kv_heads);
    const int pos = tok_pos[t], seq = tok_seq[t];
    int lo = 0;
    if (window > 0 && pos + 1 > window) lo = pos + 1 - window;
    for (int i = tid; i < hd; i += blockDim.x) qs[i] = to_f32<TQ>(q[(long long)t * q_stride + (long long)h * hd + i]);
    __syncthreads();
    float m = -INFINITY, l = 0.f, acc0 = 0.f, acc1 = 0.f;
    for (int c0 = lo; c0 <= pos; c0 += CHUNK) {
        const int n = min(CHUNK, pos + 1 - c0);
        float cmax = -INFINITY;
        for (int j = tid; j < n; j += blockDim.x) {
            const TC* kr = kc + paged_offset(c, seq, c0 + j, kvh);
            float s = 0.f;
            for (int i = 0; i < hd; ++i) s = fmaf(qs[i], to_f32<TC>(kr[i]), s);
            s *= scale;
            sc[j] = s;
            cmax = fmaxf(cmax, s);
        }
        cmax = block_max(cmax, red);
        const float m_new = fmaxf(m, cmax);
        const float corr = expf(m - m_new);          // 0 when m is -inf
        float psum = 0.f;
        for (int j = tid; j < n; j += blockDim.x) {
            const float p = expf(sc[j] - m_new);
            sc[j] = p;
            psum += p;
        }
        psum = block_sum(psum, red);                 // also orders the writes of sc before the reads
        l = l * corr + psum;
        m = m_new;
        acc0 *= corr;
        acc1 *= corr;
        for (int j = 0; j < n; ++j) {
            const TC* vr = vc + paged_offset(c, seq, c0 + j, kvh);
            const float p = sc[j];
            if (tid < hd) acc0 = fmaf(p, to_f32<TC>(vr[tid]), acc0);
            if (tid + 128 < hd) acc1 = fmaf(p, to_f32<TC>(vr[tid + 128]), acc1);
        }
        __syncthreads();
    }
    const float inv = 1.0f / l;
    TQ* o = out + (long long)t * o_stride + (long long)h * hd;
    if (tid < hd) o[tid] = from_f32<TQ>(acc0 * inv);
    if (tid + 128 < hd) o[tid + 128] = from_f32<TQ>(acc1 * inv);
}

// q: [T, *] with row stride q_stride (elements), heads side by side; out likewise.
UB_API int ub_attn_simple(const void* q, long long q_stride, int act_dtype, const void* kcache,
                          const void* vcache, int cache_dtype, void* out, long long o_stride,
                          const int* tok_pos, const int* tok_seq, const int* table, int pages_per_seq,
                          int ring, int page, int n_tokens, int nh, int nkv, int hd, int window,
                          float scale, cudaStream_t st) {
    if (n_tokens <= 0) return 0;
    if (hd > 256 || hd <= 0 || nh % nkv != 0 || ring % page != 0 || nh > 65535) return UB_ERR_ARG;
    PagedKV c{table, pages_per_seq, ring, page, nkv, hd};
    dim3 grid(n_tokens, nh);
    const size_t sm = (size_t)(hd + CHUNK) * sizeof(float);
#define GO(TQ, TC) attn_simple_kernel<TQ, TC><<<grid, 128, sm, st>>>((const TQ*)q, q_stride, (const TC*)kcache, \
        (const TC*)vcache, (TQ*)out, o_stride, tok_pos, tok_seq, c, nh, window, scale)
    if (act_dtype == UB_F32 && cache_dtype == UB_F32) GO(float, float);
    else if (act_dtype == UB_BF16 && cache_dtype == UB_BF16) GO(__nv_bfloat16, __nv_bfloat16);
    else if (act_dtype == UB_F32 && cache_dtype == UB_BF16) GO(float, __nv_bfloat16);
    else return UB_ERR_UNSUPPORTED;
#undef GO
    UB_LAUNCH_CHECK();
    return 0;
}
