// Row-wise and element-wise kernels: embedding, RMSNorm, per-head norm + rotation + cache
// write, SiLU-gate product, type conversion, random fill.
//
// Each restates one step of the reference's CPU forward pass for a whole ragged batch:
//   embedding row read        src/model/qwen_model.cpp:145-157
//   RMSNorm                   src/kernels/rmsnorm.cpp:10-17
//   per-head norm of q and k  src/model/qwen_block.cpp:76-82, :713-718
//   rotation of pairs         src/kernels/rope.cpp:17-52 (half-split or interleaved pairs, the first rope_dim columns)
//   cache write before read   src/model/qwen_block.cpp:725-727
//   silu(gate) * up           src/kernels/elementwise.cpp:62-68
// Sums of squares, the rotation and the gate are computed in 32-bit whatever the storage.
#include "common.cuh"

// ---------------------------------------------------------------------------------------
// embedding: x[t, :] = float(table[ids[t], :]); a bad id sets *status and writes zeros
// ---------------------------------------------------------------------------------------
template <typename TT>
__global__ void embed_kernel(const TT* __restrict__ table, const int* __restrict__ ids,
                             float* __restrict__ x, int width, int vocab, int* status) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const int id = ids[t];
    const bool ok = id >= 0 && id < vocab;
    if (!ok && threadIdx.x == 0) atomicExch(status, 1);
    const TT* row = table + (long long)(ok ? id : 0) * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x)
        x[(long long)t * width + i] = ok ? to_f32<TT>(row[i]) : 0.f;
}

// The same, eight values a thread and step: rows that begin on 16-byte boundaries.
template <typename TT>
__global__ void embed_vec_kernel(const TT* __restrict__ table, const int* __restrict__ ids,
                                 float* __restrict__ x, int width, int vocab, int* status) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const int id = ids[t];
    const bool ok = id >= 0 && id < vocab;
    if (!ok && threadIdx.x == 0) atomicExch(status, 1);
    const TT* row = table + (long long)(ok ? id : 0) * width;
    for (int i = threadIdx.x * 8; i < width; i += blockDim.x * 8) {
        float v[8];
        load_vec<TT, 8>(row + i, v);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = ok ? v[j] : 0.f;
        store_vec<float, 8>(x + (long long)t * width + i, v);
    }
}

UB_API int ub_embed(const void* table, int table_dtype, const int* ids, float* x, int n_tokens,
                    int width, int vocab, int* status, cudaStream_t st) {
    if (n_tokens <= 0) return 0;
    cudaError_t e;
    if (width % 8 == 0 && (((uintptr_t)table | (uintptr_t)x) & 15) == 0 && (table_dtype == UB_F32 || table_dtype == UB_BF16)) {
        int vt = 32;
        while (vt < 256 && vt * 16 < width) vt <<= 1;
        if (table_dtype == UB_F32)
            e = ub_launch_dependent(embed_vec_kernel<float>, dim3(n_tokens), dim3(vt), 0, st, (const float*)table, ids, x, width, vocab, status);
        else
            e = ub_launch_dependent(embed_vec_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(vt), 0, st, (const __nv_bfloat16*)table, ids, x, width, vocab, status);
        return (int)e;
    }
    const int threads = width >= 1024 ? 256 : 128;
    if (table_dtype == UB_F32)
        e = ub_launch_dependent(embed_kernel<float>, dim3(n_tokens), dim3(threads), 0, st, (const float*)table, ids, x, width, vocab, status);
    else if (table_dtype == UB_BF16)
        e = ub_launch_dependent(embed_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(threads), 0, st, (const __nv_bfloat16*)table, ids, x, width, vocab, status);
    else return UB_ERR_UNSUPPORTED;
    return (int)e;
}

// ---------------------------------------------------------------------------------------
// RMSNorm of rows of a float32 matrix; ``rows`` (optional) picks the input rows
// ---------------------------------------------------------------------------------------
template <typename TO>
__global__ void rmsnorm_kernel(const float* __restrict__ x, const int* __restrict__ rows,
                               const float* __restrict__ w, TO* __restrict__ out, int width, float eps) {
    __shared__ float red[33];
    pdl_trigger();
    pdl_wait();
    const int r = blockIdx.x;
    const float* xr = x + (long long)(rows ? rows[r] : r) * width;
    float ss = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) { const float v = xr[i]; ss += v * v; }
    ss = block_sum(ss, red);
    const float inv = inv_rms(ss, (float)width, eps);
    for (int i = threadIdx.x; i < width; i += blockDim.x)
        out[(long long)r * width + i] = from_f32<TO>(xr[i] * w[i] * inv);
}

// The same with rows held in registers: width a multiple of 4, at most 16 values a thread.
template <typename TO>
__global__ void rmsnorm_vec_kernel(const float* __restrict__ x, const int* __restrict__ rows,
                                   const float* __restrict__ w, TO* __restrict__ out, int width, float eps) {
    __shared__ float red[33];
    pdl_trigger();
    // the weights and the row index are there before the kernel that writes x has ended
    const int r = blockIdx.x;
    const int nv = width >> 2;
    const float4* w4 = reinterpret_cast<const float4*>(w);
    float4 g[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
        const int i = threadIdx.x + u * blockDim.x;
        if (i < nv) g[u] = w4[i];
    }
    const float4* xr = reinterpret_cast<const float4*>(x + (long long)(rows ? rows[r] : r) * width);
    pdl_wait();
    float4 v[4];
    float ss = 0.f;
#pragma unroll
    for (int u = 0; u < 4; ++u) {
        const int i = threadIdx.x + u * blockDim.x;
        if (i < nv) { v[u] = xr[i]; ss += v[u].x * v[u].x + v[u].y * v[u].y + v[u].z * v[u].z + v[u].w * v[u].w; }
    }
    ss = block_sum(ss, red);
    const float inv = inv_rms(ss, (float)width, eps);
#pragma unroll
    for (int u = 0; u < 4; ++u) {
        const int i = threadIdx.x + u * blockDim.x;
        if (i < nv) {
            const float o[4] = {v[u].x * g[u].x * inv, v[u].y * g[u].y * inv, v[u].z * g[u].z * inv, v[u].w * g[u].w * inv};
            store_vec<TO, 4>(out + (long long)r * width + 4 * i, o);
        }
    }
}

UB_API int ub_rmsnorm(const float* x, const int* rows, const float* w, void* out, int out_dtype,
                      int n_rows, int width, float eps, cudaStream_t st) {
    if (n_rows <= 0) return 0;
    cudaError_t e;
    const bool aligned = (((uintptr_t)x | (uintptr_t)w | (uintptr_t)out) & 15) == 0;
    if (width % 4 == 0 && aligned && width <= 16 * 1024) {
        int threads = 128;
        while (threads < 1024 && threads * 16 < width) threads <<= 1;
        if (width >= 2048 && threads < 256) threads = 256;
        if (out_dtype == UB_F32)
            e = ub_launch_dependent(rmsnorm_vec_kernel<float>, dim3(n_rows), dim3(threads), 0, st, x, rows, w, (float*)out, width, eps);
        else if (out_dtype == UB_BF16)
            e = ub_launch_dependent(rmsnorm_vec_kernel<__nv_bfloat16>, dim3(n_rows), dim3(threads), 0, st, x, rows, w, (__nv_bfloat16*)out, width, eps);
        else return UB_ERR_UNSUPPORTED;
        return (int)e;
    }
    const int threads = width >= 2048 ? 512 : (width >= 512 ? 256 : 128);
    if (out_dtype == UB_F32)
        e = ub_launch_dependent(rmsnorm_kernel<float>, dim3(n_rows), dim3(threads), 0, st, x, rows, w, (float*)out, width, eps);
    else if (out_dtype == UB_BF16)
        e = ub_launch_dependent(rmsnorm_kernel<__nv_bfloat16>, dim3(n_rows), dim3(threads), 0, st, x, rows, w, (__nv_bfloat16*)out, width, eps);
    else return UB_ERR_UNSUPPORTED;
    return (int)e;
}

// ---------------------------------------------------------------------------------------
// per-head norm (optional) + rotation (optional) of q and k, and the write of k and v into
// the paged cache.  One warp for each (token, head) of the fused [q | k | v] row.
//   qkv   [parts][T, (nh + 2 nkv) * hd]   the row is the sum of ``n_parts`` partial results
//                                         (slices of K of the projection), ``part_stride`` apart
//   q_out [T, *] row stride q_out_stride  normed and rotated q heads (may be qkv itself)
//   cos, sin  [max_pos, rd/2] float32 (null: no rotation); rd = ``rotary_dim`` <= hd: the head's
//             first rd columns are rotated, the others pass through (the reference's rope_dim,
//             src/kernels/rope.cpp:27,50); pairs are (j, j + rd/2), or (2j, 2j + 1) when
//             ``interleaved`` (the pairing is per-architecture data in the reference,
//             include/ultima/model/arch_registry.hpp:32-38)
//   qw, kw    [hd] float32 (null: no norm)
//   k_out, v_out  [T, nkv * hd] row stride kv_out_stride, element type of q_out (null: keys and
//             values go into the paged cache): for a position encoding that is applied by code of
//             its own between this kernel and the cache write (ub_kv_write)
// ---------------------------------------------------------------------------------------
template <typename TA, typename TQ, typename TC>
__global__ void qk_prepare_kernel(const TA* qkv, int n_parts, long long part_stride,
                                  TQ* q_out, long long q_out_stride, const float* __restrict__ qw,
                                  const float* __restrict__ kw, const float* __restrict__ cs,
                                  const float* __restrict__ sn, const int* __restrict__ tok_pos,
                                  const int* __restrict__ tok_seq, TC* __restrict__ kcache,
                                  TC* __restrict__ vcache, PagedKV c, int n_tokens, int nh, float eps,
                                  int write_kv, int rd, int interleaved, TQ* k_out, TQ* v_out, long long kv_out_stride) {
    pdl_trigger();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const long long wid = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int heads_all = nh + 2 * c.n_kv_heads;
    if (wid >= (long long)n_tokens * heads_all) return;
    const int t = (int)(wid / heads_all), h = (int)(wid % heads_all);
    const int hd = c.head_dim, n_pairs = hd >> 1, rhalf = rd >> 1;
    const TA* row = qkv + ((long long)t * heads_all + h) * hd;
    const int pos = tok_pos[t];
    const int seq = tok_seq[t];
    if (h >= nh + c.n_kv_heads) {                       // a value head: copy into the cache (or to v_out)
        if (!write_kv) return;
        const int kvh = h - nh - c.n_kv_heads;
        TC* dst = v_out ? nullptr : vcache + paged_offset(c, seq, pos, kvh);
        TQ* dst2 = v_out ? v_out + (long long)t * kv_out_stride + (long long)kvh * hd : nullptr;
        for (int i = lane; i < hd; i += 32) {
            float v = 0.f;
            for (int p = 0; p < n_parts; ++p) v += to_f32<TA>(row[p * part_stride + i]);
            if (dst2) dst2[i] = from_f32<TQ>(v); else dst[i] = from_f32<TC>(v);
        }
        return;
    }
    const bool is_k = h >= nh;
    if (is_k && !write_kv) return;
    const float* w = is_k ? kw : qw;
    // a lane's pairs: pair x for x = lane, lane + 32, ...: at most 4 (head sizes up to 256).  The
    // first rd/2 pairs are the rotated ones, the rest are neighbours that pass through.
    float va[4], vb[4];
    int ia[4], ib[4];
    float ss = 0.f;
#pragma unroll
    for (int u = 0; u < 4; ++u) {
        const int x = lane + u * 32;
        va[u] = vb[u] = 0.f;
        ia[u] = ib[u] = 0;
        if (x < n_pairs) {
            if (x < rhalf) { ia[u] = interleaved ? 2 * x : x; ib[u] = interleaved ? 2 * x + 1 : x + rhalf; }
            else { ia[u] = rd + 2 * (x - rhalf); ib[u] = ia[u] + 1; }
            for (int p = 0; p < n_parts; ++p) {
                va[u] += to_f32<TA>(row[p * part_stride + ia[u]]);
                vb[u] += to_f32<TA>(row[p * part_stride + ib[u]]);
            }
            ss += va[u] * va[u] + vb[u] * vb[u];
        }
    }
    ss = warp_sum(ss);
    const float inv = w ? inv_rms(ss, (float)hd, eps) : 1.0f;
    TC* dst = (is_k && !k_out) ? kcache + paged_offset(c, seq, pos, h - nh) : nullptr;
    TQ* qdst = is_k ? (k_out ? k_out + (long long)t * kv_out_stride + (long long)(h - nh) * hd : nullptr)
                    : q_out + (long long)t * q_out_stride + (long long)h * hd;
#pragma unroll
    for (int u = 0; u < 4; ++u) {
        const int x = lane + u * 32;
        if (x >= n_pairs) continue;
        float a = va[u], b = vb[u];
        if (w) { a = a * w[ia[u]] * inv; b = b * w[ib[u]] * inv; }
        float ra = a, rb = b;
        if (cs && x < rhalf) {
            const float co = cs[(long long)pos * rhalf + x], si = sn[(long long)pos * rhalf + x];
            ra = a * co - b * si;
            rb = a * si + b * co;
        }
        if (dst) { dst[ia[u]] = from_f32<TC>(ra); dst[ib[u]] = from_f32<TC>(rb); }
        else { qdst[ia[u]] = from_f32<TQ>(ra); qdst[ib[u]] = from_f32<TQ>(rb); }
    }
}

// Rotation alone, in place: x [T, n_heads, hd] (token stride x_stride elements, heads side by side),
// the tables and the pairing as above.  One warp a (token, head).
template <typename TX>
__global__ void rotate_pairs_kernel(TX* x, long long x_stride, int n_tokens, int n_heads, int hd, const float* __restrict__ cs,
                                    const float* __restrict__ sn, const int* __restrict__ tok_pos, int rd, int interleaved) {
    const int lane = threadIdx.x & 31;
    const long long wid = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (wid >= (long long)n_tokens * n_heads) return;
    const int t = (int)(wid / n_heads), h = (int)(wid % n_heads);
    const int rhalf = rd >> 1;
    TX* row = x + (long long)t * x_stride + (long long)h * hd;
    const int pos = tok_pos[t];
    for (int j = lane; j < rhalf; j += 32) {
        const int ia = interleaved ? 2 * j : j, ib = interleaved ? 2 * j + 1 : j + rhalf;
        const float a = to_f32<TX>(row[ia]), b = to_f32<TX>(row[ib]);
        const float co = cs[(long long)pos * rhalf + j], si = sn[(long long)pos * rhalf + j];
        row[ia] = from_f32<TX>(a * co - b * si);
        row[ib] = from_f32<TX>(a * si + b * co);
    }
}
UB_API int ub_rotate_pairs(void* x, int dtype, long long x_stride, int n_tokens, int n_heads, int hd, const float* cs,
                           const float* sn, const int* tok_pos, int rotary_dim, int interleaved, cudaStream_t st) {
    if (n_tokens <= 0 || n_heads <= 0) return 0;
    if (rotary_dim < 2 || rotary_dim % 2 != 0 || rotary_dim > hd || !cs || !sn) return UB_ERR_ARG;
    const long long warps = (long long)n_tokens * n_heads;
    const unsigned grid = (unsigned)((warps + 7) / 8);
    if (dtype == UB_F32) rotate_pairs_kernel<float><<<grid, 256, 0, st>>>((float*)x, x_stride, n_tokens, n_heads, hd, cs, sn, tok_pos, rotary_dim, interleaved);
    else if (dtype == UB_BF16) rotate_pairs_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((__nv_bfloat16*)x, x_stride, n_tokens, n_heads, hd, cs, sn, tok_pos, rotary_dim, interleaved);
    else return UB_ERR_UNSUPPORTED;
    UB_LAUNCH_CHECK();
    return 0;
}

// Keys and values of the step's tokens, k and v [T, nkv * hd] (row stride kv_stride), into the paged
// cache.  One warp a (token, kv head).
template <typename TX, typename TC>
__global__ void kv_write_kernel(const TX* __restrict__ k, const TX* __restrict__ v, long long kv_stride, const int* __restrict__ tok_pos,
                                const int* __restrict__ tok_seq, TC* __restrict__ kcache, TC* __restrict__ vcache, PagedKV c,
                                int n_tokens) {
    const int lane = threadIdx.x & 31;
    const long long wid = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (wid >= (long long)n_tokens * c.n_kv_heads) return;
    const int t = (int)(wid / c.n_kv_heads), h = (int)(wid % c.n_kv_heads);
    const long long at = paged_offset(c, tok_seq[t], tok_pos[t], h);
    const TX* kr = k + (long long)t * kv_stride + (long long)h * c.head_dim;
    const TX* vr = v + (long long)t * kv_stride + (long long)h * c.head_dim;
    for (int i = lane; i < c.head_dim; i += 32) {
        kcache[at + i] = from_f32<TC>(to_f32<TX>(kr[i]));
        vcache[at + i] = from_f32<TC>(to_f32<TX>(vr[i]));
    }
}
UB_API int ub_kv_write(const void* k, const void* v, int dtype, long long kv_stride, const int* tok_pos, const int* tok_seq,
                       void* kcache, void* vcache, int cache_dtype, const int* table, int pages_per_seq, int ring, int page,
                       int n_tokens, int nkv, int hd, cudaStream_t st) {
    if (n_tokens <= 0) return 0;
    if (ring % page != 0 || nkv < 1 || hd < 1) return UB_ERR_ARG;
    PagedKV c{table, pages_per_seq, ring, page, nkv, hd};
    const unsigned grid = (unsigned)(((long long)n_tokens * nkv + 7) / 8);
    if (dtype == UB_F32 && cache_dtype == UB_F32)
        kv_write_kernel<float, float><<<grid, 256, 0, st>>>((const float*)k, (const float*)v, kv_stride, tok_pos, tok_seq, (float*)kcache, (float*)vcache, c, n_tokens);
    else if (dtype == UB_BF16 && cache_dtype == UB_BF16)
        kv_write_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)k, (const __nv_bfloat16*)v, kv_stride, tok_pos, tok_seq, (__nv_bfloat16*)kcache, (__nv_bfloat16*)vcache, c, n_tokens);
    else if (dtype == UB_F32 && cache_dtype == UB_BF16)
        kv_write_kernel<float, __nv_bfloat16><<<grid, 256, 0, st>>>((const float*)k, (const float*)v, kv_stride, tok_pos, tok_seq, (__nv_bfloat16*)kcache, (__nv_bfloat16*)vcache, c, n_tokens);
    else return UB_ERR_UNSUPPORTED;
    UB_LAUNCH_CHECK();
    return 0;
}

// The same for head sizes of 64, 128 and 256.  Sixteen lanes take a head: a lane holds E = hd / 32
// neighbouring elements of the head's first half and the E elements of the second half that pair with
// them in the rotation, so the rotation needs no exchange between lanes, the sum of squares four, and
// every access is one aligned vector.  Two heads a warp and instruction mean half as many instructions a
// byte as a head a warp, which is what this kernel is short of (its loads are small and many).
template <typename TA, typename TQ, typename TC, int E>
__global__ void __launch_bounds__(256, 3) qk_prepare_vec_kernel(const TA* qkv, int n_parts, long long part_stride,
                                      TQ* q_out, long long q_out_stride, const float* __restrict__ qw,
                                      const float* __restrict__ kw, const float* __restrict__ cs,
                                      const float* __restrict__ sn, const int* __restrict__ tok_pos,
                                      const int* __restrict__ tok_seq, TC* __restrict__ kcache,
                                      TC* __restrict__ vcache, PagedKV c, int n_tokens, int nh, float eps,
                                      int write_kv) {
    pdl_trigger();
    // blockIdx.x is the token; the half-warps of its blocks take the token's heads in turn, so what
    // belongs to the token (its position, the cosines and sines of that position, the norm weights) is
    // fetched once a lane, and before the kernel that writes qkv has ended: none of it is written by a kernel
    const int hl = threadIdx.x & 15, hw = threadIdx.x >> 4, n_hw = blockDim.x >> 4;
    const int heads_all = nh + 2 * c.n_kv_heads;
    const int t = blockIdx.x;
    constexpr int hd = 32 * E, half = hd / 2;
    const int pos = tok_pos[t];
    const int seq = tok_seq[t];
    float co[E], si[E], gq[2][E], gk[2][E];
    if (qw) { load_vec<float, E>(qw + hl * E, gq[0]); load_vec<float, E>(qw + half + hl * E, gq[1]); }
    if (kw) { load_vec<float, E>(kw + hl * E, gk[0]); load_vec<float, E>(kw + half + hl * E, gk[1]); }
    // where the token's keys and values go: the page is looked up once, a head is then a stride away
    const int li = pos % c.ring;
    const long long kv_at = write_kv ? (((long long)c.table[(long long)seq * c.pages_per_seq + li / c.page] * c.n_kv_heads) * c.page
                                        + (li % c.page)) * hd + hl * E : 0;
    const long long kv_head_stride = (long long)c.page * hd;
    const TA* trow = qkv + (long long)t * heads_all * hd + hl * E;
    TQ* qrow = q_out + (long long)t * q_out_stride + hl * E;
    pdl_wait();
    // three of the half-warp's heads at a time (all of them where a token has up to 48 heads and its block
    // sixteen half-warps): their loads are in flight before the first is used
    constexpr int UH = 3;
    const int h_step = n_hw * gridDim.y;
    // (the loop's count is the same for both halves of a warp: they meet in the shuffles below)
    const int h_first = blockIdx.y * n_hw + (hw & ~1);
    for (int hb = h_first; hb < heads_all; hb += UH * h_step) {
        const int h0 = hb + (hw & 1);
        float v3[UH][2][E];
#pragma unroll
        for (int u = 0; u < UH; ++u) {
            const int h = h0 + u * h_step;
            const bool is_kv = h >= nh;
            if (h < heads_all && !(is_kv && !write_kv)) {
                load_vec<TA, E>(trow + h * hd, v3[u][0]);
                load_vec<TA, E>(trow + h * hd + half, v3[u][1]);
            }
        }
        if (cs && hb == h_first) {
            // after the first heads' loads, which do not have to wait for the position as these do
            load_vec<float, E>(cs + (long long)pos * half + hl * E, co);
            load_vec<float, E>(sn + (long long)pos * half + hl * E, si);
        }
#pragma unroll
        for (int u = 0; u < UH; ++u) {
            const int h = h0 + u * h_step;
            // (a half-warp whose head is past the last one still takes part in the shuffles below)
            const bool live = h < heads_all;
            const bool is_v = h >= nh + c.n_kv_heads, is_k = !is_v && h >= nh;
            const bool skip = !live || ((is_v || is_k) && !write_kv);
            float (*v)[E] = v3[u];
            if (!skip) {
                const TA* row = trow + h * hd;
                for (int p = 1; p < n_parts; ++p) {
                    float more[2][E];
                    load_vec<TA, E>(row + p * part_stride, more[0]);
                    load_vec<TA, E>(row + p * part_stride + half, more[1]);
#pragma unroll
                    for (int i = 0; i < E; ++i) { v[0][i] += more[0][i]; v[1][i] += more[1][i]; }
                }
            }
            if (!skip && is_v) {
                TC* dst = vcache + kv_at + (h - nh - c.n_kv_heads) * kv_head_stride;
                store_vec<TC, E>(dst, v[0]);
                store_vec<TC, E>(dst + half, v[1]);
            }
            const bool normed = is_k ? kw != nullptr : qw != nullptr;
            float ss = 0.f;
            if (!skip && !is_v && normed) {
#pragma unroll
                for (int i = 0; i < E; ++i) ss += v[0][i] * v[0][i] + v[1][i] * v[1][i];
            }
            // the sum over the sixteen lanes of the head (all lanes of the warp take part)
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            if (skip || is_v) continue;
            if (normed) {
                const float inv = inv_rms(ss, (float)hd, eps);
#pragma unroll
                for (int i = 0; i < E; ++i) {
                    v[0][i] = v[0][i] * (is_k ? gk[0][i] : gq[0][i]) * inv;
                    v[1][i] = v[1][i] * (is_k ? gk[1][i] : gq[1][i]) * inv;
                }
            }
            if (cs) {
#pragma unroll
                for (int i = 0; i < E; ++i) {
                    const float a = v[0][i], b = v[1][i];
                    v[0][i] = a * co[i] - b * si[i];
                    v[1][i] = a * si[i] + b * co[i];
                }
            }
            if (is_k) {
                TC* dst = kcache + kv_at + (h - nh) * kv_head_stride;
                store_vec<TC, E>(dst, v[0]);
                store_vec<TC, E>(dst + half, v[1]);
            } else {
                store_vec<TQ, E>(qrow + h * hd, v[0]);
                store_vec<TQ, E>(qrow + h * hd + half, v[1]);
            }
        }
    }
}

UB_API int ub_qk_prepare(const void* qkv, int in_dtype, int n_parts, long long part_stride, void* q_out,
                         int q_dtype, long long q_out_stride, const float* qw, const float* kw, const float* cs,
                         const float* sn, const int* tok_pos, const int* tok_seq, void* kcache,
                         void* vcache, int cache_dtype, const int* table, int pages_per_seq, int ring,
                         int page, int n_tokens, int nh, int nkv, int hd, float eps, int write_kv,
                         int rotary_dim, int interleaved, void* k_out, void* v_out, long long kv_out_stride,
                         cudaStream_t st) {
    if (n_tokens <= 0) return 0;
    if (hd % 2 != 0 || hd > 256 || ring % page != 0 || n_parts < 1) return UB_ERR_ARG;
    if (cs && (rotary_dim < 2 || rotary_dim % 2 != 0 || rotary_dim > hd)) return UB_ERR_ARG;
    if ((!k_out) != (!v_out)) return UB_ERR_ARG;
    if (!cs) { rotary_dim = 0; interleaved = 0; }
    PagedKV c{table, pages_per_seq, ring, page, nkv, hd};
    const long long warps = (long long)n_tokens * (nh + 2 * nkv);
    const int wpb = 8;
    const unsigned grid = (unsigned)((warps + wpb - 1) / wpb);
    cudaError_t e;
    const bool aligned = (((uintptr_t)qkv | (uintptr_t)q_out | (uintptr_t)kcache | (uintptr_t)vcache | (uintptr_t)qw |
                           (uintptr_t)kw | (uintptr_t)cs | (uintptr_t)sn) & 15) == 0 &&
                         part_stride % 8 == 0 && q_out_stride % 8 == 0;
    // the vector kernel: whole heads rotated in halves, keys and values straight into the cache
    const bool vec = aligned && (hd == 64 || hd == 128 || hd == 256) && !k_out && (!cs || (rotary_dim == hd && !interleaved));
    // blocks of 16 half-warps; with many tokens one block a token (its half-warps loop over the heads), with
    // few tokens a half-warp a head
    const int heads_all = nh + 2 * nkv;
    const dim3 vgrid(n_tokens, n_tokens >= 256 ? 1 : (heads_all + 15) / 16);
#define LAUNCH_V(TA, TQ, TC, E) e = ub_launch_dependent(qk_prepare_vec_kernel<TA, TQ, TC, E>, vgrid, dim3(256), 0, st, \
        (const TA*)qkv, n_parts, part_stride, (TQ*)q_out, q_out_stride, qw, kw, cs, sn, tok_pos, tok_seq, \
        (TC*)kcache, (TC*)vcache, c, n_tokens, nh, eps, write_kv)
#define LAUNCH(TA, TQ, TC) do { \
        if (vec && hd == 64) LAUNCH_V(TA, TQ, TC, 2); else if (vec && hd == 128) LAUNCH_V(TA, TQ, TC, 4); \
        else if (vec && hd == 256) LAUNCH_V(TA, TQ, TC, 8); \
        else e = ub_launch_dependent(qk_prepare_kernel<TA, TQ, TC>, dim3(grid), dim3(wpb * 32), 0, st, \
        (const TA*)qkv, n_parts, part_stride, (TQ*)q_out, q_out_stride, qw, kw, cs, sn, tok_pos, tok_seq, \
        (TC*)kcache, (TC*)vcache, c, n_tokens, nh, eps, write_kv, rotary_dim, interleaved, (TQ*)k_out, (TQ*)v_out, \
        kv_out_stride); } while (0)
    if (in_dtype == UB_F32 && q_dtype == UB_F32 && cache_dtype == UB_F32) LAUNCH(float, float, float);
    else if (in_dtype == UB_BF16 && q_dtype == UB_BF16 && cache_dtype == UB_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16, __nv_bfloat16);
    else if (in_dtype == UB_F32 && q_dtype == UB_BF16 && cache_dtype == UB_BF16) LAUNCH(float, __nv_bfloat16, __nv_bfloat16);
    else if (in_dtype == UB_F32 && q_dtype == UB_F32 && cache_dtype == UB_BF16) LAUNCH(float, float, __nv_bfloat16);
    else return UB_ERR_UNSUPPORTED;
#undef LAUNCH
#undef LAUNCH_V
    return (int)e;
}

// ---------------------------------------------------------------------------------------
// out[t, f] = silu(gu[t, f]) * gu[t, F + f]   (gate and up side by side in one row)
// ---------------------------------------------------------------------------------------
template <typename TI, typename TO>
__global__ void silu_mul_kernel(const TI* __restrict__ gu, int n_parts, long long part_stride, TO* __restrict__ out,
                                long long n, int F) {
    pdl_trigger();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const long long t = i / F;
    const int f = (int)(i % F);
    float g = 0.f, u = 0.f;
    for (int p = 0; p < n_parts; ++p) {
        g += to_f32<TI>(gu[p * part_stride + t * 2 * F + f]);
        u += to_f32<TI>(gu[p * part_stride + t * 2 * F + F + f]);
    }
    out[i] = from_f32<TO>(g / (1.0f + expf(-g)) * u);
}

// gu: [parts][T, 2F], the sum of the parts is [gate | up]
UB_API int ub_silu_mul(const void* gu, int in_dtype, int n_parts, long long part_stride, void* out, int out_dtype,
                       int n_tokens, int F, cudaStream_t st) {
    const long long n = (long long)n_tokens * F;
    if (n <= 0) return 0;
    if (n_parts < 1) return UB_ERR_ARG;
    const unsigned grid = (unsigned)((n + 255) / 256);
    cudaError_t e;
#define LAUNCH(TI, TO) e = ub_launch_dependent(silu_mul_kernel<TI, TO>, dim3(grid), dim3(256), 0, st, (const TI*)gu, n_parts, part_stride, (TO*)out, n, F)
    if (in_dtype == UB_F32 && out_dtype == UB_F32) LAUNCH(float, float);
    else if (in_dtype == UB_F32 && out_dtype == UB_BF16) LAUNCH(float, __nv_bfloat16);
    else if (in_dtype == UB_BF16 && out_dtype == UB_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
    else return UB_ERR_UNSUPPORTED;
#undef LAUNCH
    return (int)e;
}

// ---------------------------------------------------------------------------------------
// conversion and accumulation: out = convert(in);  acc += in
// ---------------------------------------------------------------------------------------
template <typename TI, typename TO>
__global__ void convert_kernel(const TI* __restrict__ in, TO* __restrict__ out, long long n) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = from_f32<TO>(to_f32<TI>(in[i]));
}
UB_API int ub_convert(const void* in, int in_dtype, void* out, int out_dtype, long long n, cudaStream_t st) {
    if (n <= 0) return 0;
    const unsigned grid = (unsigned)((n + 255) / 256);
    if (in_dtype == UB_F32 && out_dtype == UB_BF16) convert_kernel<float, __nv_bfloat16><<<grid, 256, 0, st>>>((const float*)in, (__nv_bfloat16*)out, n);
    else if (in_dtype == UB_BF16 && out_dtype == UB_F32) convert_kernel<__nv_bfloat16, float><<<grid, 256, 0, st>>>((const __nv_bfloat16*)in, (float*)out, n);
    else if (in_dtype == UB_F32 && out_dtype == UB_F32) convert_kernel<float, float><<<grid, 256, 0, st>>>((const float*)in, (float*)out, n);
    else if (in_dtype == UB_BF16 && out_dtype == UB_BF16) convert_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)in, (__nv_bfloat16*)out, n);
    else return UB_ERR_UNSUPPORTED;
    UB_LAUNCH_CHECK();
    return 0;
}

template <typename TI>
__global__ void add_into_kernel(float* __restrict__ acc, const TI* __restrict__ in, long long n) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) acc[i] += to_f32<TI>(in[i]);
}
UB_API int ub_add_into(float* acc, const void* in, int in_dtype, long long n, cudaStream_t st) {
    if (n <= 0) return 0;
    const unsigned grid = (unsigned)((n + 255) / 256);
    if (in_dtype == UB_F32) add_into_kernel<float><<<grid, 256, 0, st>>>(acc, (const float*)in, n);
    else if (in_dtype == UB_BF16) add_into_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(acc, (const __nv_bfloat16*)in, n);
    else return UB_ERR_UNSUPPORTED;
    UB_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------------------------------
// random fill: out[i] = shift + std * z(key, i), z standard normal.
//
// One counter-based generator, written three times with the same bits: here, in numpy in
// weights/random_init.py and, as the tests' own copy, in tests/plain_random.py.  A draw depends on
// the tensor's key and the element's index only.  Every step is an integer operation or ONE
// correctly rounded float32 operation (add, multiply, divide, square root; never a fused
// multiply-add, never a library logarithm or cosine), so the three give the same bits:
//   r  = mix64(key ^ mix64(i))                        SplitMix64's finaliser
//   u1 = ((r >> 41) + 0.5) * 2^-23                    in (0, 1), exact
//   t  = (r >> 16) & 0xFFFFFF                          24 bits: the angle 2 pi t / 2^24
//   ln u1   exponent * ln 2 + 2 s (1 + s^2/3 + ... + s^10/11), s = (m - 1) / (m + 1), m the
//           mantissa brought into [sqrt(1/2), sqrt(2))
//   cos     quadrant from the top two bits of t, the rest folded into [0, pi/4], Taylor sums of
//           sine and cosine there (to x^9 and x^10), Horner's rule
//   z  = sqrt(-2 ln u1) * cos(2 pi t / 2^24)          Box-Muller
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ unsigned long long mix64(unsigned long long z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
__device__ __forceinline__ float fbits(unsigned u) { return __uint_as_float(u); }
__device__ __forceinline__ float counter_normal(unsigned long long key, unsigned long long i) {
    const unsigned long long r = mix64(key ^ mix64(i));
    // ---- ln(u1)
    const float u1 = __fmul_rn(__fadd_rn(__uint2float_rn((unsigned)(r >> 41)), 0.5f), fbits(0x34000000u));   // * 2^-23
    const unsigned ub = __float_as_uint(u1);
    int e = (int)(ub >> 23) - 127;
    float m = fbits((ub & 0x7FFFFFu) | 0x3F800000u);                  // [1, 2)
    if (m > fbits(0x3FB504F3u)) { m = __fmul_rn(m, 0.5f); e += 1; }    // [sqrt(1/2), sqrt(2))
    const float s = __fdiv_rn(__fsub_rn(m, 1.0f), __fadd_rn(m, 1.0f));
    const float s2 = __fmul_rn(s, s);
    float p = fbits(0x3DBA2E8Cu);                                      // 1/11
    p = __fadd_rn(__fmul_rn(p, s2), fbits(0x3DE38E39u));               // 1/9
    p = __fadd_rn(__fmul_rn(p, s2), fbits(0x3E124925u));               // 1/7
    p = __fadd_rn(__fmul_rn(p, s2), fbits(0x3E4CCCCDu));               // 1/5
    p = __fadd_rn(__fmul_rn(p, s2), fbits(0x3EAAAAABu));               // 1/3
    p = __fadd_rn(__fmul_rn(p, s2), 1.0f);
    const float ln_m = __fmul_rn(__fmul_rn(2.0f, s), p);
    const float ln_u = __fadd_rn(__fmul_rn(__int2float_rn(e), fbits(0x3F317218u)), ln_m);    // e ln 2 + ln m
    const float rad = __fsqrt_rn(__fmul_rn(-2.0f, ln_u));
    // ---- cos(2 pi t / 2^24)
    const unsigned t = (unsigned)(r >> 16) & 0xFFFFFFu;
    const unsigned quad = t >> 22, rest = t & 0x3FFFFFu;              // angle = (quad + rest / 2^22) pi/2
    const bool fold = rest > 0x200000u;                                // past the middle of the quadrant
    const unsigned fr = fold ? 0x400000u - rest : rest;               // [0, 2^21]
    const float x = __fmul_rn(__fmul_rn(__uint2float_rn(fr), fbits(0x34800000u)), fbits(0x3FC90FDBu));   // * 2^-22 * pi/2
    const float x2 = __fmul_rn(x, x);
    float sn = fbits(0x3638EF1Du);                                     // 1/9!
    sn = __fsub_rn(fbits(0x39500D01u), __fmul_rn(sn, x2));             // 1/7! - ...
    sn = __fsub_rn(fbits(0x3C088889u), __fmul_rn(sn, x2));             // 1/5! - ...
    sn = __fsub_rn(fbits(0x3E2AAAABu), __fmul_rn(sn, x2));             // 1/3! - ...
    sn = __fsub_rn(1.0f, __fmul_rn(sn, x2));
    sn = __fmul_rn(sn, x);
    float cs = fbits(0x3493F27Eu);                                     // 1/10!
    cs = __fsub_rn(fbits(0x37D00D01u), __fmul_rn(cs, x2));             // 1/8! - ...
    cs = __fsub_rn(fbits(0x3AB60B61u), __fmul_rn(cs, x2));             // 1/6! - ...
    cs = __fsub_rn(fbits(0x3D2AAAABu), __fmul_rn(cs, x2));             // 1/4! - ...
    cs = __fsub_rn(0.5f, __fmul_rn(cs, x2));
    cs = __fsub_rn(1.0f, __fmul_rn(cs, x2));
    const float sin_q = fold ? cs : sn, cos_q = fold ? sn : cs;        // sine and cosine of the angle within the quadrant
    const float c = quad == 0 ? cos_q : quad == 1 ? -sin_q : quad == 2 ? -cos_q : sin_q;
    return __fmul_rn(rad, c);
}
template <typename TO>
__global__ void fill_normal_kernel(TO* __restrict__ out, long long n, unsigned long long key, float shift, float stdv) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    out[i] = from_f32<TO>(__fadd_rn(shift, __fmul_rn(stdv, counter_normal(key, (unsigned long long)i))));
}
UB_API int ub_fill_normal(void* out, int dtype, long long n, unsigned long long seed, float shift, float stdv,
                          cudaStream_t st) {
    if (n <= 0) return 0;
    const unsigned grid = (unsigned)((n + 255) / 256);
    if (dtype == UB_F32) fill_normal_kernel<float><<<grid, 256, 0, st>>>((float*)out, n, seed, shift, stdv);
    else if (dtype == UB_BF16) fill_normal_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((__nv_bfloat16*)out, n, seed, shift, stdv);
    else return UB_ERR_UNSUPPORTED;
    UB_LAUNCH_CHECK();
    return 0;
}
