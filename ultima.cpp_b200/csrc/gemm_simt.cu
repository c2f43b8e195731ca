// Matrix product on the CUDA cores, any sizes, any mix of float32 and bfloat16 operands,
// float32 FMA accumulation in k order: out[t, n] = sum_k A[t, k] * W[n, k].
//
// This is the true 32-bit path of every projection (no tensor-core mode that rounds its
// inputs), and the fallback for shapes the tensor-core kernel refuses.  It restates the
// reference's batched product, one weight row reused across tokens
// (src/model/weight_dispatch.cpp:374-441, src/kernels/dot_batched.cpp:39-96).
// The k order of every output's sum is the same whatever the number of rows, so a token's
// result does not depend on what else is in the batch.
#include "common.cuh"

enum : int { EPI_STORE = 0, EPI_ADD = 1, EPI_SWIGLU = 2 };

constexpr int BM = 64, BN = 64, BK = 16;

template <typename TA, typename TW, typename TO, int EPI>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const TA* __restrict__ A, const TW* __restrict__ W, const TW* __restrict__ W2,
                 TO* __restrict__ out, int M, int N, int K, long long lda, long long ldw, long long ldo) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    __shared__ float W2s[EPI == EPI_SWIGLU ? BK : 1][BN + 4];
    const int tid = threadIdx.x;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int tm = (tid / 16) * 4, tn = (tid % 16) * 4;
    float acc[4][4] = {}, acc2[4][4] = {};
    for (int k0 = 0; k0 < K; k0 += BK) {
        // 64 x 16 elements of each operand, 4 for each thread
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int e = tid + i * 256;
            const int r = e / BK, kk = e % BK;
            const int k = k0 + kk;
            float a = 0.f, w = 0.f, w2 = 0.f;
            if (k < K) {
                if (m0 + r < M) a = to_f32<TA>(A[(long long)(m0 + r) * lda + k]);
                if (n0 + r < N) {
                    w = to_f32<TW>(W[(long long)(n0 + r) * ldw + k]);
                    if (EPI == EPI_SWIGLU) w2 = to_f32<TW>(W2[(long long)(n0 + r) * ldw + k]);
                }
            }
            As[kk][r] = a;
            Ws[kk][r] = w;
            if (EPI == EPI_SWIGLU) W2s[kk][r] = w2;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[4], b[4], b2[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) { a[i] = As[kk][tm + i]; b[i] = Ws[kk][tn + i]; }
            if (EPI == EPI_SWIGLU) {
#pragma unroll
                for (int i = 0; i < 4; ++i) b2[i] = W2s[kk][tn + i];
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
                    if (EPI == EPI_SWIGLU) acc2[i][j] = fmaf(a[i], b2[j], acc2[i][j]);
                }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + tm + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tn + j;
            if (n >= N) continue;
            TO* p = out + (long long)m * ldo + n;
            if (EPI == EPI_STORE) *p = from_f32<TO>(acc[i][j]);
            else if (EPI == EPI_ADD) *p = from_f32<TO>(to_f32<TO>(*p) + acc[i][j]);
            else { const float g = acc[i][j]; *p = from_f32<TO>(g / (1.0f + expf(-g)) * acc2[i][j]); }
        }
    }
}

template <typename TA, typename TW, typename TO>
static int launch(const void* A, const void* W, const void* W2, void* out, int M, int N, int K,
                  long long lda, long long ldw, long long ldo, int epi, cudaStream_t st) {
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    if (grid.y > 65535) return UB_ERR_ARG;
#define GO(E) gemm_simt_kernel<TA, TW, TO, E><<<grid, 256, 0, st>>>((const TA*)A, (const TW*)W, (const TW*)W2, (TO*)out, M, N, K, lda, ldw, ldo)
    if (epi == EPI_STORE) GO(EPI_STORE);
    else if (epi == EPI_ADD) GO(EPI_ADD);
    else if (epi == EPI_SWIGLU) { if (!W2) return UB_ERR_ARG; GO(EPI_SWIGLU); }
    else return UB_ERR_ARG;
#undef GO
    UB_LAUNCH_CHECK();
    return 0;
}

// a_dtype, w_dtype, o_dtype: UB_F32 / UB_BF16.  EPI_ADD needs a float32 output.
UB_API int ub_gemm_simt(const void* A, int a_dtype, const void* W, const void* W2, int w_dtype, void* out,
                        int o_dtype, int M, int N, int K, long long lda, long long ldw, long long ldo,
                        int epi, cudaStream_t st) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0) return UB_ERR_ARG;
    if (epi == EPI_ADD && o_dtype != UB_F32) return UB_ERR_ARG;
    const int key = a_dtype * 4 + w_dtype * 2 + o_dtype;
    switch (key) {
        case 0: return launch<float, float, float>(A, W, W2, out, M, N, K, lda, ldw, ldo, epi, st);
        case 1: return launch<float, float, __nv_bfloat16>(A, W, W2, out, M, N, K, lda, ldw, ldo, epi, st);
        case 2: return launch<float, __nv_bfloat16, float>(A, W, W2, out, M, N, K, lda, ldw, ldo, epi, st);
        case 3: return launch<float, __nv_bfloat16, __nv_bfloat16>(A, W, W2, out, M, N, K, lda, ldw, ldo, epi, st);
        case 4: return launch<__nv_bfloat16, float, float>(A, W, W2, out, M, N, K, lda, ldw, ldo, epi, st);
        case 5: return launch<__nv_bfloat16, float, __nv_bfloat16>(A, W, W2, out, M, N, K, lda, ldw, ldo, epi, st);
        case 6: return launch<__nv_bfloat16, __nv_bfloat16, float>(A, W, W2, out, M, N, K, lda, ldw, ldo, epi, st);
        case 7: return launch<__nv_bfloat16, __nv_bfloat16, __nv_bfloat16>(A, W, W2, out, M, N, K, lda, ldw, ldo, epi, st);
    }
    return UB_ERR_UNSUPPORTED;
}
