// Plain attention over the paged cache, for prefill and decode alike.
//
// One block per (token, query head).  The token at position p of sequence b sees the cached
// keys lo..p of that sequence (itself included: its key was written before this kernel runs),
// lo = 0, or p - window + 1 for a windowed layer.  Query head h reads kv head h / (nq / nkv).
// Scores, the running maximum, the exponentials, their sum and the weighted sum of values are
// float32.  This is the 32-bit path and the twin the fast kernels are checked against; it
// restates ops.AttentionScoresInto (pkg/ops/attention.go:10-47) and replaces the reference's
// attn_qk / softmax / attn_v PTX kernels (pkg/gpu/cuda/ptx.go:679-889), which the host loops
// over heads.
#include "common.cuh"

#define ATT_WARPS 4
#define ATT_MAXD 256

template <typename T>
__global__ void __launch_bounds__(ATT_WARPS * 32) attention_plain_kernel(
    const T* q, const T* k_pool, const T* v_pool, T* __restrict__ out,
    const int* __restrict__ positions, const int* __restrict__ seq_of_token,
    const int* __restrict__ page_table, int max_pages, int page_size,
    int nq, int nkv, int d, float scale, int window, const PageBounds pb) {
    pdl_launch();
    pdl_wait();
    extern __shared__ float sm[];
    float* qs = sm;                       // [d]
    float* accs = sm + d;                 // [ATT_WARPS][d]
    float* ml = accs + ATT_WARPS * d;     // [ATT_WARPS][2]
    const int t = blockIdx.x, h = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    T* o = out + ((size_t)t * nq + h) * d;
    const int b = seq_of_token[t];
    if (b < 0) {
        for (int i = threadIdx.x; i < d; i += blockDim.x) o[i] = from_f<T>(0.f);
        return;
    }
    const int pos = positions[t];
    const int g = h / (nq / nkv);
    int lo = 0;
    if (window > 0 && pos - window + 1 > 0) lo = pos - window + 1;
    const T* qp = q + ((size_t)t * nq + h) * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x) qs[i] = to_f<T>(qp[i]);
    __syncthreads();

    float acc[ATT_MAXD / 32];
#pragma unroll
    for (int j = 0; j < ATT_MAXD / 32; ++j) acc[j] = 0.f;
    float m = -INFINITY, l = 0.f;
    const int* pt = page_table + (size_t)b * max_pages;
    for (int j = lo + warp; j <= pos; j += ATT_WARPS) {
        const int page = gg_page(pt, j / page_size, max_pages, pb, 41);
        const size_t base = (((size_t)page * nkv + g) * page_size + (j % page_size)) * d;
        const T* kp = k_pool + base;
        const T* vp = v_pool + base;
        float dot = 0.f;
        for (int i = lane; i < d; i += 32) dot = fmaf(qs[i], to_f<T>(kp[i]), dot);
        dot = warp_sum(dot) * scale;
        const float mn = fmaxf(m, dot);
        const float corr = expf(m - mn);
        const float p = expf(dot - mn);
        l = l * corr + p;
#pragma unroll
        for (int jj = 0; jj < ATT_MAXD / 32; ++jj) {
            const int i = lane + 32 * jj;
            if (i < d) acc[jj] = acc[jj] * corr + p * to_f<T>(vp[i]);
        }
        m = mn;
    }
#pragma unroll
    for (int jj = 0; jj < ATT_MAXD / 32; ++jj) {
        const int i = lane + 32 * jj;
        if (i < d) accs[warp * d + i] = acc[jj];
    }
    if (lane == 0) { ml[warp * 2] = m; ml[warp * 2 + 1] = l; }
    __syncthreads();
    float M = -INFINITY;
    for (int w = 0; w < ATT_WARPS; ++w) M = fmaxf(M, ml[w * 2]);
    float L = 0.f;
    float f[ATT_WARPS];
    for (int w = 0; w < ATT_WARPS; ++w) { f[w] = expf(ml[w * 2] - M); L += ml[w * 2 + 1] * f[w]; }
    const float inv = 1.0f / L;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        float s = 0.f;
        for (int w = 0; w < ATT_WARPS; ++w) s += accs[w * d + i] * f[w];
        o[i] = from_f<T>(s * inv);
    }
}

// q[T, nq, d] and out[T, nq, d] in `dtype`; pools [page][nkv][page_size][d] in `dtype`, n_pages of them.
// status (may be null): where the debug build records a page id or table index out of range (code 41).
GG_API gg_attention_plain(const void* q, const void* k_pool, const void* v_pool, void* out, int dtype,
                          const int* positions, const int* seq_of_token, const int* page_table,
                          int max_pages, int page_size, int n_pages, int ntok, int nq, int nkv, int d,
                          float scale, int window, int* status, cudaStream_t stream) {
    if (ntok <= 0) return 0;
    if (d <= 0 || d > ATT_MAXD || nq <= 0 || nkv <= 0 || nq % nkv || nq > 65535 || page_size <= 0) return GG_ERR_ARG;
    const size_t smem = ((size_t)(1 + ATT_WARPS) * d + 2 * ATT_WARPS) * sizeof(float);
    dim3 grid(ntok, nq);
    GG_DISPATCH_DTYPE(dtype, T,
        gg_launch(attention_plain_kernel<T>, dim3(grid), dim3(ATT_WARPS * 32), smem, stream, 1, 
            (const T*)q, (const T*)k_pool, (const T*)v_pool, (T*)out, positions, seq_of_token, page_table,
            max_pages, page_size, nq, nkv, d, scale, window, PageBounds{n_pages, status}));
    return gg_last_error();
}

// 1 if this library was built with checked page tables (the debug build), else 0.
GG_API gg_attention_plain_checked() { return gg_debug_bounds(); }
