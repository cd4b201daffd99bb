// Row-wise and element-wise kernels: embedding gather, RMSNorm, rotary tables,
// fused per-head QK-norm + rotary + cache write, SwiGLU, residual add, row statistics.
//
// They replace the reference's rmsnorm / rope_heads / swiglu / add_inplace PTX
// kernels (pkg/gpu/cuda/ptx.go:428-496, 498-564, 634-677, 891-924), which run
// one vector per launch; these run every token of a step in one launch.
// Reductions, the inverse root, the rotation and the SiLU are done in float32
// (angles in float64); the residual stream is float32 in both precisions.
#include "common.cuh"

// ----------------------------------------------------------------------------- embedding
template <typename TW>
__global__ void embed_gather_kernel(const TW* __restrict__ table, const int* tokens,
                                    float* __restrict__ out, int H, int V) {
    pdl_launch();
    pdl_wait();
    const int t = blockIdx.x;
    const int tok = tokens[t];
    float* o = out + (size_t)t * H;
    if (tok < 0 || tok >= V) {  // padding row
        for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = 0.f;
        return;
    }
    const TW* r = table + (size_t)tok * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = to_f<TW>(r[i]);
}

GG_API gg_embed_gather(const void* table, int table_dtype, const int* tokens, float* out,
                       int T, int H, int V, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (H <= 0 || V <= 0) return GG_ERR_ARG;
    GG_DISPATCH_DTYPE(table_dtype, TW,
        gg_launch(embed_gather_kernel<TW>, dim3(T), dim3(256), 0, stream, 1, (const TW*)table, tokens, out, H, V));
    return gg_last_error();
}

// ----------------------------------------------------------------------------- RMSNorm
// out[r,:] = x[src(r),:] * (1/sqrt(mean(x^2)+eps)) * w ; src(r) = rows ? rows[r] : r.
// x is the float32 residual stream.  A negative source row gives a zero row.
template <typename TO>
__global__ void rmsnorm_kernel(const float* x, const int* __restrict__ rows,
                               const float* __restrict__ w, TO* __restrict__ out, int H, float eps) {
    pdl_launch();
    pdl_wait();
    __shared__ float red[33];
    const int r = blockIdx.x;
    const int src = rows ? rows[r] : r;
    TO* o = out + (size_t)r * H;
    if (src < 0) {
        for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = from_f<TO>(0.f);
        return;
    }
    const float* xr = x + (size_t)src * H;
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) { float v = xr[i]; ss = fmaf(v, v, ss); }
    ss = block_sum(ss, red);
    const float scale = 1.0f / sqrtf(ss / (float)H + eps);
    for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = from_f<TO>(xr[i] * scale * w[i]);
}

// Same result for rows of up to 8192 floats whose length is a multiple of 4: the row is read once with
// 16-byte loads that are all in flight together and kept in registers for the second pass.  In a
// decode step only a few rows exist, so the kernel's time is one memory latency, not two loops of them.
template <typename TO, int VPT /* float4 per thread */>
__global__ void __launch_bounds__(256) rmsnorm_vec_kernel(const float* x, const int* __restrict__ rows,
                                                          const float* __restrict__ w, TO* __restrict__ out, int H, float eps) {
    pdl_launch();
    pdl_wait();
    __shared__ float red[33];
    const int r = blockIdx.x;
    const int src = rows ? rows[r] : r;
    TO* o = out + (size_t)r * H;
    const int nvec = H >> 2;
    float4 v[VPT];
    float ss = 0.f;
    if (src >= 0) {
        const float4* xr = reinterpret_cast<const float4*>(x + (size_t)src * H);
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            const int i = threadIdx.x + j * 256;
            v[j] = i < nvec ? xr[i] : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            ss = fmaf(v[j].x, v[j].x, ss); ss = fmaf(v[j].y, v[j].y, ss);
            ss = fmaf(v[j].z, v[j].z, ss); ss = fmaf(v[j].w, v[j].w, ss);
        }
    } else {
#pragma unroll
        for (int j = 0; j < VPT; ++j) v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    ss = block_sum(ss, red);
    const float scale = src >= 0 ? 1.0f / sqrtf(ss / (float)H + eps) : 0.f;
    const float4* wr = reinterpret_cast<const float4*>(w);
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
        const int i = threadIdx.x + j * 256;
        if (i < nvec) {
            const float4 ww = wr[i];
            const float a = v[j].x * scale * ww.x, b = v[j].y * scale * ww.y;
            const float c = v[j].z * scale * ww.z, d = v[j].w * scale * ww.w;
            if (sizeof(TO) == 4) {
                reinterpret_cast<float4*>(o)[i] = make_float4(a, b, c, d);
            } else {
                __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
                uint2 pk;
                pk.x = *reinterpret_cast<uint32_t*>(&lo);
                pk.y = *reinterpret_cast<uint32_t*>(&hi);
                reinterpret_cast<uint2*>(o)[i] = pk;
            }
        }
    }
}

GG_API gg_rmsnorm(const float* x, const int* rows, const float* w, void* out, int out_dtype,
                  int R, int H, float eps, cudaStream_t stream) {
    if (R <= 0) return 0;
    if (H <= 0) return GG_ERR_ARG;
    const bool aligned = (H % 4 == 0) && ((((uintptr_t)x) & 15) == 0) && ((((uintptr_t)w) & 15) == 0) &&
                         ((((uintptr_t)out) & 15) == 0);
    if (aligned && H <= 8192) {
        const int vpt = (H / 4 + 255) / 256;     // 1..8
        GG_DISPATCH_DTYPE(out_dtype, TO, {
            if (vpt <= 1) gg_launch(rmsnorm_vec_kernel<TO, 1>, dim3(R), dim3(256), 0, stream, 1, x, rows, w, (TO*)out, H, eps);
            else if (vpt <= 2) gg_launch(rmsnorm_vec_kernel<TO, 2>, dim3(R), dim3(256), 0, stream, 1, x, rows, w, (TO*)out, H, eps);
            else if (vpt <= 4) gg_launch(rmsnorm_vec_kernel<TO, 4>, dim3(R), dim3(256), 0, stream, 1, x, rows, w, (TO*)out, H, eps);
            else gg_launch(rmsnorm_vec_kernel<TO, 8>, dim3(R), dim3(256), 0, stream, 1, x, rows, w, (TO*)out, H, eps);
        });
        return gg_last_error();
    }
    const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
    GG_DISPATCH_DTYPE(out_dtype, TO,
        gg_launch(rmsnorm_kernel<TO>, dim3(R), dim3(threads), 0, stream, 1, x, rows, w, (TO*)out, H, eps));
    return gg_last_error();
}

// ----------------------------------------------------------------------------- row statistics
// What a product with a folded RMSNorm reads instead of the normalised rows: xhat = bfloat16(x) and,
// per row, the sums of squares over blocks of 128 columns (ceil(H / 128) partial sums).  The products
// that add into the residual stream write both themselves; this kernel makes them where no such
// product came before (after the embedding, after a part that does not emit them).
__global__ void __launch_bounds__(128) row_stats_kernel(const float* x, bf16* __restrict__ xhat,
                                                        float* __restrict__ ssq, int H, int parts) {
    pdl_launch();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int part = blockIdx.y * 4 + (threadIdx.x >> 5);
    const int t = blockIdx.x;
    if (part >= parts) return;
    const int c0 = part * 128 + lane * 4;
    const float* xr = x + (size_t)t * H + c0;
    bf16* hr = xhat + (size_t)t * H + c0;
    float ss = 0.f;
    if (c0 + 4 <= H && ((((uintptr_t)xr) & 15) == 0) && ((((uintptr_t)hr) & 7) == 0)) {
        const float4 v = *reinterpret_cast<const float4*>(xr);
        ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
        __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
        *reinterpret_cast<uint2*>(hr) = make_uint2(*reinterpret_cast<uint32_t*>(&a), *reinterpret_cast<uint32_t*>(&b));
    } else {
        for (int j = 0; j < 4; ++j)
            if (c0 + j < H) { const float v = xr[j]; ss = fmaf(v, v, ss); hr[j] = __float2bfloat16_rn(v); }
    }
    ss = warp_sum(ss);
    if (lane == 0) ssq[(size_t)t * parts + part] = ss;
}

GG_API gg_row_stats(const float* x, void* xhat, float* ssq, int T, int H, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (H <= 0 || H > 128 * 4 * 65535) return GG_ERR_ARG;
    const int parts = (H + 127) / 128;
    gg_launch(row_stats_kernel, dim3(T, (parts + 3) / 4), dim3(128), 0, stream, 1, x, (bf16*)xhat, ssq, H, parts);
    return gg_last_error();
}

// ----------------------------------------------------------------------------- rotary tables
// cos/sin[t, i] of angle = pos[t] * inv_freq[i], computed in float64 (the reference computes
// its tables in float64 too, pkg/ops/rope_tables.go:6-20) and stored as float32.
__global__ void rope_tables_kernel(const int* __restrict__ positions, const double* __restrict__ inv_freq,
                                   float* __restrict__ cosv, float* __restrict__ sinv, int T, int half) {
    pdl_launch();
    pdl_wait();
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= T * half) return;
    const int t = idx / half, i = idx - t * half;
    int p = positions[t];
    if (p < 0) p = 0;
    double s, c;
    sincos((double)p * inv_freq[i], &s, &c);
    cosv[idx] = (float)c;
    sinv[idx] = (float)s;
}

GG_API gg_rope_tables(const int* positions, const double* inv_freq, float* cosv, float* sinv,
                      int T, int half, cudaStream_t stream) {
    if (T <= 0 || half <= 0) return 0;
    const int n = T * half;
    gg_launch(rope_tables_kernel, dim3((n + 255) / 256), dim3(256), 0, stream, 1, positions, inv_freq, cosv, sinv, T, half);
    return gg_last_error();
}

// ----------------------------------------------------------------------------- QK-norm + rotary + cache write
// One warp per (token, head) of the fused projection output qkv[T, (nq + 2 nkv) * d]:
//   q heads: optional RMSNorm over d with weight qw, rotary, written to q_out[T, nq, d];
//   k heads: optional RMSNorm with kw, rotary, written into the paged key pool;
//   v heads: copied into the paged value pool.
// Order as in the reference: norm first, rotation after (pkg/model/qwen3/model.go:227-236).
// Pool layout: [page][kv_head][page_size][d]; the page of position p of sequence b is
// page_table[b * max_pages + p / page_size].  Pools may be null (a layer that reads another
// layer's cache writes none); then k and v heads are skipped.
template <typename T>
__global__ void qk_norm_rope_cache_kernel(
    const T* qkv, T* __restrict__ q_out,
    const float* __restrict__ qw, const float* __restrict__ kw, float eps,
    const float* cosv, const float* sinv,
    const int* __restrict__ positions, const int* __restrict__ seq_of_token,
    const int* __restrict__ page_table, int max_pages, int page_size,
    T* __restrict__ k_pool, T* __restrict__ v_pool,
    int ntok, int nq, int nkv, int d, int rot, const PageBounds pb) {
    pdl_launch();
    pdl_wait();
    extern __shared__ float sm[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nheads = nq + 2 * nkv;
    const long long wid = (long long)blockIdx.x * (blockDim.x >> 5) + warp;
    if (wid >= (long long)ntok * nheads) return;
    const int t = (int)(wid / nheads), h = (int)(wid - (long long)t * nheads);
    const int b = seq_of_token[t];
    const bool is_q = h < nq, is_k = !is_q && h < nq + nkv;
    if (!is_q && (k_pool == nullptr || b < 0)) return;
    float* buf = sm + warp * d;
    const T* src = qkv + ((size_t)t * nheads + h) * d;
    T* dst;
    if (is_q) {
        dst = q_out + ((size_t)t * nq + h) * d;
    } else {
        const int pos = positions[t];
        const int page = gg_page_w(page_table + (size_t)b * max_pages, pos / page_size, max_pages, pb, 46);
        if (page < 0) return;            // (debug build) outside the pool: nothing is written
        const int kvh = is_k ? h - nq : h - nq - nkv;
        T* pool = is_k ? k_pool : v_pool;
        dst = pool + (((size_t)page * nkv + kvh) * page_size + (pos % page_size)) * d;
    }
    if (!is_q && !is_k) {  // value head: plain copy
        for (int i = lane; i < d; i += 32) dst[i] = src[i];
        return;
    }
    const float* w = is_q ? qw : kw;
    float ss = 0.f;
    for (int i = lane; i < d; i += 32) { float v = to_f<T>(src[i]); buf[i] = v; ss = fmaf(v, v, ss); }
    float scale = 1.f;
    if (w != nullptr) {
        ss = warp_sum(ss);
        scale = 1.0f / sqrtf(ss / (float)d + eps);
    }
    __syncwarp();
    const int half = rot >> 1;
    const float* c = cosv + (size_t)t * half;
    const float* s = sinv + (size_t)t * half;
    for (int i = lane; i < d; i += 32) {
        float v = buf[i] * scale * (w ? w[i] : 1.f);
        float o;
        if (i < half) {
            const float p = buf[i + half] * scale * (w ? w[i + half] : 1.f);
            o = v * c[i] - p * s[i];
        } else if (i < rot) {
            const int j = i - half;
            const float p = buf[j] * scale * (w ? w[j] : 1.f);
            o = p * s[j] + v * c[j];
        } else {
            o = v;
        }
        dst[i] = from_f<T>(o);
    }
}

// bfloat16 form for a full rotation (rot == d) and d = 64, 128 or 256.  D / 16 lanes share one head: a lane
// owns eight pairs (i, i + d/2), i = 8 * sub .. + 8, so both halves of a pair sit in the same thread and
// every access to the head is 16 bytes wide; a warp handles 32 / (D / 16) heads at once (four of size 128),
// which keeps 1 KB in flight per warp.  The head's sum of squares is added over its lanes by shuffles.
template <int D>
__global__ void __launch_bounds__(128) qk_norm_rope_cache_vec_kernel(
    const bf16* qkv, bf16* __restrict__ q_out,
    const float* __restrict__ qw, const float* __restrict__ kw, float eps,
    const float* cosv, const float* sinv,
    const int* __restrict__ positions, const int* __restrict__ seq_of_token,
    const int* __restrict__ page_table, int max_pages, int page_size,
    bf16* __restrict__ k_pool, bf16* __restrict__ v_pool, int ntok, int nq, int nkv, const PageBounds pb) {
    pdl_launch();
    pdl_wait();
    constexpr int HALF = D / 2, LPH = D / 16, HPW = 32 / LPH;      // lanes per head, heads per warp
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nheads = nq + 2 * nkv;
    const long long item = ((long long)blockIdx.x * (blockDim.x >> 5) + warp) * HPW + lane / LPH;
    const int sub = lane % LPH;
    const bool in_range = item < (long long)ntok * nheads;
    const int t = in_range ? (int)(item / nheads) : 0, h = in_range ? (int)(item - (long long)t * nheads) : 0;
    const int b = in_range ? seq_of_token[t] : -1;
    const bool is_q = h < nq, is_k = !is_q && h < nq + nkv;
    bool live = in_range && (is_q || (k_pool != nullptr && b >= 0));     // every lane stays for the shuffles
    const bf16* src = qkv + ((size_t)t * nheads + h) * D;
    bf16* dst = nullptr;
    if (live) {
        if (is_q) {
            dst = q_out + ((size_t)t * nq + h) * D;
        } else {
            const int pos = positions[t];
            const int page = gg_page_w(page_table + (size_t)b * max_pages, pos / page_size, max_pages, pb, 47);
            const int kvh = is_k ? h - nq : h - nq - nkv;
            if (page < 0) live = false;      // (debug build) outside the pool: nothing is written
            else dst = (is_k ? k_pool : v_pool) + (((size_t)page * nkv + kvh) * page_size + (pos % page_size)) * D;
        }
    }
    const int i0 = sub * 8;             // first index of this lane in the low half
    uint4 lo4 = make_uint4(0, 0, 0, 0), hi4 = make_uint4(0, 0, 0, 0);
    if (live) {
        lo4 = *reinterpret_cast<const uint4*>(src + i0);
        hi4 = *reinterpret_cast<const uint4*>(src + i0 + HALF);
    }
    if (live && !is_q && !is_k) {       // value head: plain copy
        *reinterpret_cast<uint4*>(dst + i0) = lo4;
        *reinterpret_cast<uint4*>(dst + i0 + HALF) = hi4;
    }
    const bool rotate = live && (is_q || is_k);
    const float* w = is_q ? qw : kw;
    float4 cs[2], sn[2], wl[2], wh[2];
    if (rotate) {                       // asked for before the sum of squares is known
        const float4* cp = reinterpret_cast<const float4*>(cosv + (size_t)t * HALF + i0);
        const float4* sp = reinterpret_cast<const float4*>(sinv + (size_t)t * HALF + i0);
        cs[0] = cp[0]; cs[1] = cp[1]; sn[0] = sp[0]; sn[1] = sp[1];
        if (w != nullptr) {
            wl[0] = reinterpret_cast<const float4*>(w + i0)[0]; wl[1] = reinterpret_cast<const float4*>(w + i0)[1];
            wh[0] = reinterpret_cast<const float4*>(w + i0 + HALF)[0]; wh[1] = reinterpret_cast<const float4*>(w + i0 + HALF)[1];
        }
    }
    const bf16* lo = reinterpret_cast<const bf16*>(&lo4);
    const bf16* hi = reinterpret_cast<const bf16*>(&hi4);
    float a[8], c[8], ss = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        a[k] = __bfloat162float(lo[k]); c[k] = __bfloat162float(hi[k]);
        ss = fmaf(a[k], a[k], ss); ss = fmaf(c[k], c[k], ss);
    }
#pragma unroll
    for (int o = LPH / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (!rotate) return;
    const float scale = w != nullptr ? 1.0f / sqrtf(ss / (float)D + eps) : 1.f;
    const float* csf = reinterpret_cast<const float*>(cs);
    const float* snf = reinterpret_cast<const float*>(sn);
    const float* wlf = reinterpret_cast<const float*>(wl);
    const float* whf = reinterpret_cast<const float*>(wh);
    uint4 olo, ohi;
    bf16* ol = reinterpret_cast<bf16*>(&olo);
    bf16* oh = reinterpret_cast<bf16*>(&ohi);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const float x0 = a[k] * scale * (w != nullptr ? wlf[k] : 1.f);
        const float x1 = c[k] * scale * (w != nullptr ? whf[k] : 1.f);
        ol[k] = __float2bfloat16_rn(x0 * csf[k] - x1 * snf[k]);
        oh[k] = __float2bfloat16_rn(x0 * snf[k] + x1 * csf[k]);
    }
    *reinterpret_cast<uint4*>(dst + i0) = olo;
    *reinterpret_cast<uint4*>(dst + i0 + HALF) = ohi;
}

GG_API gg_qk_norm_rope_cache(const void* qkv, int dtype, void* q_out, const float* qw, const float* kw, float eps,
                             const float* cosv, const float* sinv, const int* positions, const int* seq_of_token,
                             const int* page_table, int max_pages, int page_size, int n_pages, void* k_pool, void* v_pool,
                             int ntok, int nq, int nkv, int d, int rot, int* status, cudaStream_t stream) {
    if (ntok <= 0) return 0;
    if (d <= 0 || d > 1024 || rot < 0 || rot > d || (rot & 1) || nq <= 0 || nkv <= 0 || page_size <= 0) return GG_ERR_ARG;
    const int warps = 4;
    const long long total = (long long)ntok * (nq + 2 * nkv);
    const unsigned grid = (unsigned)((total + warps - 1) / warps);
    const bool al = ((((uintptr_t)qkv) | ((uintptr_t)q_out) | ((uintptr_t)k_pool) | ((uintptr_t)v_pool) |
                      ((uintptr_t)cosv) | ((uintptr_t)sinv) | ((uintptr_t)qw) | ((uintptr_t)kw)) & 15) == 0;
    if (dtype == GG_BF16 && rot == d && al && (d == 64 || d == 128 || d == 256)) {
        const int per_block = warps * (32 / (d / 16));          // heads a block of four warps handles
        const unsigned vgrid = (unsigned)((total + per_block - 1) / per_block);
#define GG_QK_VEC(D_) gg_launch(qk_norm_rope_cache_vec_kernel<D_>, dim3(vgrid), dim3(warps * 32), 0, stream, 1,  \
            (const bf16*)qkv, (bf16*)q_out, qw, kw, eps, cosv, sinv, positions, seq_of_token, page_table, max_pages, \
            page_size, (bf16*)k_pool, (bf16*)v_pool, ntok, nq, nkv, PageBounds{n_pages, status})
        if (d == 64) GG_QK_VEC(64); else if (d == 128) GG_QK_VEC(128); else GG_QK_VEC(256);
#undef GG_QK_VEC
        return gg_last_error();
    }
    const size_t smem = (size_t)warps * d * sizeof(float);
    GG_DISPATCH_DTYPE(dtype, T,
        gg_launch(qk_norm_rope_cache_kernel<T>, dim3(grid), dim3(warps * 32), smem, stream, 1, 
            (const T*)qkv, (T*)q_out, qw, kw, eps, cosv, sinv, positions, seq_of_token, page_table, max_pages,
            page_size, (T*)k_pool, (T*)v_pool, ntok, nq, nkv, d, rot, PageBounds{n_pages, status}));
    return gg_last_error();
}

// ----------------------------------------------------------------------------- SwiGLU
// out[t, i] = silu(gu[t, i]) * gu[t, I + i], silu(z) = z / (1 + exp(-z)) (pkg/ops/ops.go:316-318).
template <typename T>
__global__ void swiglu_kernel(const T* gu, T* __restrict__ out, long long n, int I) {
    pdl_launch();
    pdl_wait();
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n) return;
    const long long t = idx / I;
    const int i = (int)(idx - t * I);
    const float g = to_f<T>(gu[t * 2 * I + i]);
    const float u = to_f<T>(gu[t * 2 * I + I + i]);
    out[idx] = from_f<T>(g / (1.0f + expf(-g)) * u);
}

// Eight elements per thread with 16-byte accesses (rows of I elements, I a multiple of 8).
__global__ void swiglu_vec8_kernel(const bf16* gu, bf16* __restrict__ out, long long nvec, int I8) {
    pdl_launch();
    pdl_wait();
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= nvec) return;
    const long long t = idx / I8;
    const int c = (int)(idx - t * I8);
    const uint4 gv = *reinterpret_cast<const uint4*>(gu + (t * 2 * I8 + c) * 8);
    const uint4 uv = *reinterpret_cast<const uint4*>(gu + (t * 2 * I8 + I8 + c) * 8);
    const uint32_t* gw = reinterpret_cast<const uint32_t*>(&gv);
    const uint32_t* uw = reinterpret_cast<const uint32_t*>(&uv);
    uint32_t ow[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const __nv_bfloat162 g2 = *reinterpret_cast<const __nv_bfloat162*>(&gw[k]);
        const __nv_bfloat162 u2 = *reinterpret_cast<const __nv_bfloat162*>(&uw[k]);
        const float g0 = __low2float(g2), g1 = __high2float(g2);
        const float r0 = g0 / (1.0f + expf(-g0)) * __low2float(u2);
        const float r1 = g1 / (1.0f + expf(-g1)) * __high2float(u2);
        const __nv_bfloat162 r = __floats2bfloat162_rn(r0, r1);
        ow[k] = *reinterpret_cast<const uint32_t*>(&r);
    }
    *reinterpret_cast<uint4*>(out + idx * 8) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
}

GG_API gg_swiglu(const void* gu, int dtype, void* out, int ntok, int I, cudaStream_t stream) {
    if (ntok <= 0) return 0;
    if (I <= 0) return GG_ERR_ARG;
    const long long n = (long long)ntok * I;
    if (dtype == GG_BF16 && I % 8 == 0 && ((((uintptr_t)gu) | ((uintptr_t)out)) & 15) == 0) {
        const long long nvec = n / 8;
        gg_launch(swiglu_vec8_kernel, dim3((unsigned)((nvec + 255) / 256)), dim3(256), 0, stream, 1, (const bf16*)gu, (bf16*)out, nvec, I / 8);
        return gg_last_error();
    }
    GG_DISPATCH_DTYPE(dtype, T,
        gg_launch(swiglu_kernel<T>, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, 1, (const T*)gu, (T*)out, n, I));
    return gg_last_error();
}

// ----------------------------------------------------------------------------- residual add
// x (float32) += delta.  The fast path folds this into the producing product's epilogue;
// this is the stand-alone form (pkg/gpu/cuda/ptx.go:891-924 add_inplace).
template <typename T>
__global__ void residual_add_kernel(float* __restrict__ x, const T* delta, long long n) {
    pdl_launch();
    pdl_wait();
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx < n) x[idx] += to_f<T>(delta[idx]);
}

GG_API gg_residual_add(float* x, const void* delta, int dtype, long long n, cudaStream_t stream) {
    if (n <= 0) return 0;
    GG_DISPATCH_DTYPE(dtype, T,
        gg_launch(residual_add_kernel<T>, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, 1, x, (const T*)delta, n));
    return gg_last_error();
}

// ----------------------------------------------------------------------------- token feed
// tokens[i] = sampled[src[i]] where src[i] >= 0: lets a decode step take the ids that the previous
// step's sampling kernel left on the device, without a round trip through the host.
__global__ void feed_tokens_kernel(int* __restrict__ tokens, const int* __restrict__ src,
                                   const int* sampled, int n) {
    pdl_launch();
    pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n && src[i] >= 0) tokens[i] = sampled[src[i]];
}

GG_API gg_feed_tokens(int* tokens, const int* src, const int* sampled, int n, cudaStream_t stream) {
    if (n <= 0) return 0;
    return gg_launch(feed_tokens_kernel, dim3((n + 127) / 128), dim3(128), 0, stream, 1, tokens, src, sampled, n);
}

// 1 if this library was built with checked page tables (the debug build), else 0.
GG_API gg_elementwise_checked() { return gg_debug_bounds(); }
