// Shared helpers of the kernels: element types, conversions, reductions, launch checks.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

#define UB_API extern "C" __attribute__((visibility("default")))

// element type codes of the C interface
enum : int { UB_F32 = 0, UB_BF16 = 1 };

// Every exported function returns 0 or a negative code for a refused argument, or the
// positive cudaError_t of a failed launch.
#define UB_ERR_ARG (-1)
#define UB_ERR_UNSUPPORTED (-2)
#define UB_LAUNCH_CHECK() do { cudaError_t e__ = cudaGetLastError(); if (e__ != cudaSuccess) return (int)e__; } while (0)

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// Programmatic dependent launch.  ``pdl_trigger`` lets a kernel that was launched as this one's
// programmatic dependent begin (it still waits for this kernel's end before it reads its inputs);
// ``pdl_wait`` is that wait.  Both do nothing in a kernel launched the ordinary way.
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Launch ``kern`` as a programmatic dependent of the kernel before it in the stream: it may begin
// while that kernel still runs, so it must call pdl_wait() before it reads or writes anything the
// earlier kernels touch, and before any thread returns.
template <typename... KArgs, typename... Args>
static inline cudaError_t ub_launch_dependent(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                              cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
}

// E consecutive elements (E * sizeof(T) bytes: 4, 8, 16 or 32, aligned to min(16, that)) to and
// from float registers.
template <typename T, int E>
__device__ __forceinline__ void load_vec(const T* p, float* out) {
    constexpr int NB = sizeof(T) * E;
    static_assert(NB == 4 || NB == 8 || NB % 16 == 0, "vector of 4, 8 or a multiple of 16 bytes");
    alignas(16) T tmp[E];
    if constexpr (NB == 4) *reinterpret_cast<uint32_t*>(tmp) = *reinterpret_cast<const uint32_t*>(p);
    else if constexpr (NB == 8) *reinterpret_cast<uint2*>(tmp) = *reinterpret_cast<const uint2*>(p);
    else {
#pragma unroll
        for (int i = 0; i < NB / 16; ++i) reinterpret_cast<uint4*>(tmp)[i] = reinterpret_cast<const uint4*>(p)[i];
    }
#pragma unroll
    for (int i = 0; i < E; ++i) out[i] = to_f32<T>(tmp[i]);
}
template <typename T, int E>
__device__ __forceinline__ void store_vec(T* p, const float* v) {
    constexpr int NB = sizeof(T) * E;
    alignas(16) T tmp[E];
    if constexpr (sizeof(T) == 2 && E % 2 == 0) {
        // two values a conversion instruction
#pragma unroll
        for (int i = 0; i < E; i += 2)
            *reinterpret_cast<__nv_bfloat162*>(&tmp[i]) = __floats2bfloat162_rn(v[i], v[i + 1]);
    } else {
#pragma unroll
        for (int i = 0; i < E; ++i) tmp[i] = from_f32<T>(v[i]);
    }
    if constexpr (NB == 4) *reinterpret_cast<uint32_t*>(p) = *reinterpret_cast<const uint32_t*>(tmp);
    else if constexpr (NB == 8) *reinterpret_cast<uint2*>(p) = *reinterpret_cast<const uint2*>(tmp);
    else {
#pragma unroll
        for (int i = 0; i < NB / 16; ++i) reinterpret_cast<uint4*>(p)[i] = reinterpret_cast<const uint4*>(tmp)[i];
    }
}

// 1 / sqrt(sum of squares / n + eps) of the norms: the hardware's reciprocal square root refined by
// one Newton step, which leaves it within an ulp or two of the division by the square root.
__device__ __forceinline__ float inv_rms(float sum_sq, float n, float eps) {
    const float x = sum_sq / n + eps;
    const float y = rsqrtf(x);
    return y * fmaf(-0.5f * x * y, y, 1.5f);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.  ``red`` holds 33 floats.
__device__ __forceinline__ float block_sum(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nw ? red[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}
__device__ __forceinline__ float block_max(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nw ? red[lane] : -INFINITY;
        t = warp_max(t);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}

// Where a sequence's position lies in a paged cache.  A sequence's pages are listed in
// ``table`` (``pages_per_seq`` entries for each sequence of the step); ``ring`` is the
// number of positions the sequence's storage holds (a multiple of the page size): a full
// cache holds all positions, a window cache wraps around.
struct PagedKV {
    const int* table;       // [n_seqs, pages_per_seq]
    int pages_per_seq;
    int ring;               // positions held for each sequence
    int page;               // positions in a page
    int n_kv_heads;
    int head_dim;
};
__device__ __forceinline__ long long paged_offset(const PagedKV& c, int seq, int pos, int kv_head) {
    const int li = pos % c.ring;
    const int pg = c.table[(long long)seq * c.pages_per_seq + li / c.page];
    return (((long long)pg * c.n_kv_heads + kv_head) * c.page + (li % c.page)) * c.head_dim;
}
