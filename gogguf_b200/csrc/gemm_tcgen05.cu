// bfloat16 matrix product on the 5th-generation tensor cores of sm_100a:
//   D[i, j] = sum_k A[i, k] * B[j, k],  A[RA, K] and B[RB, K] both K-major, float32 accumulate.
//
// One CTA computes one 128 x BN tile of D over a slab of K:
//   * warp 0, one thread: TMA producer.  cp.async.bulk.tensor loads a [128 x 64] tile of A and a
//     [BN x 64] tile of B per pipeline stage into 128-byte-swizzled shared memory and signals the
//     stage's "full" mbarrier with the byte count.
//   * warp 1, one thread: issues tcgen05.mma (kind::f16, M = 128, N = BN, K = 16) four times per
//     stage with the accumulator in tensor memory, then tcgen05.commit to the stage's "empty"
//     mbarrier (frees the stage when the tensor core has read it) and, after the last stage, to
//     the "accumulator ready" mbarrier.  Warp 1 also allocates and frees the tensor memory.
//   * warps 2..5: epilogue.  tcgen05.ld brings the accumulator to registers (each warp its own 32
//     lanes of tensor memory), converts and stores.
//
// Two orientations share the kernel.  Prefill ("normal"): A = activations x[M, K], B = weights
// W[N, K], out[m, n] = D[m, n].  Decode ("swap"): A = weights, so that the 128-row side of the
// instruction is filled by output features and a small batch of tokens is the N side (16..128);
// out[m, n] = D[n, m].  In decode the product is a stream of weights from HBM: the grid is
// widened by splitting K over blockIdx.z and several CTAs share an SM.  The CTAs that hold the
// partial sums of one output tile form a thread-block cluster: each dumps its accumulator into its
// own shared memory, and every CTA adds one slice of the tile over all ranks through distributed
// shared memory, always in rank order, and writes it out (up to 16 tokens the slices are sent with
// st.async and counted by an mbarrier of the receiver, so no cluster barrier stands at the end of
// the kernel; above that cluster barriers frame the exchange).  No scratch memory, no second
// launch, no float atomics: results do not depend on timing.  (A second form
// keeps the partial sums in a float32 scratch buffer in global memory and adds them in a second
// kernel; it serves callers that ask for it and split counts beyond a cluster.)
//
// Further down in this file: the persistent prefill forms (one CTA per SM on 128 x 256 tiles, and CTA pairs
// on 256 x 256 tiles with cta_group::2, which split K over work items when a product has fewer tiles than
// pairs), and what the epilogues fuse: the residual add, SwiGLU over interleaved gate/up rows, an RMSNorm
// folded in on either side (NormIO), and for the q/k/v product (decode form and CTA pairs) the per-head norm,
// the rotation and the cache write (QkvIO).
//
// Every mbarrier wait is bounded; a wait that runs out records a code in the status word, raises
// the CTA's abort flag, and all roles fall through to the common exit, which lets copies in flight
// land and frees the tensor memory.
//
// The reference multiplies with a one-thread-per-row scalar PTX kernel (pkg/gpu/cuda/ptx.go:67-129).
#include <cuda.h>
#include <type_traits>
#include "common.cuh"
#include "tma_util.cuh"

namespace {

constexpr int BM = 128;           // rows of A per tile = MMA M
constexpr int BK = 64;            // bf16 elements per stage row = 128 bytes = one swizzle atom
constexpr int UMMA_K = 16;
constexpr int A_BYTES = BM * BK * 2;
constexpr int NUM_THREADS = 192;

enum OutMode { OUT_BF16 = 0, OUT_F32 = 1, OUT_F32_ACC = 2, OUT_SWIGLU = 3, OUT_QKV = 4 };

// mbarrier, TMA and tcgen05 wrappers: one set for every kernel of the package (tma_util.cuh)
using tma::smem_u32;
using tma::mbar_init;
using tma::mbar_expect_tx;
using tma::mbar_arrive;
using tma::mbar_try_wait;
using tma::mbar_wait;
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
    tma::load_2d(dst, map, bar, x, y);
}
// K-major tile with rows of 128 bytes, 128-byte swizzle: 8-row groups are 1024 bytes apart
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr) { return tc5::smem_desc(saddr, 16, 1024); }
// kind::f16: bf16 x bf16 -> f32, both operands K-major
__device__ __forceinline__ uint32_t make_idesc(int m, int n) { return tc5::idesc_bf16(m, n, 0); }
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
    tc5::mma(tmem_d, adesc, bdesc, idesc, acc);
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) { tc5::commit(bar); }
__device__ __forceinline__ void tc_fence_before() { tc5::fence_before(); }
__device__ __forceinline__ void tc_fence_after() { tc5::fence_after(); }
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t* r) { tc5::ld16(taddr, r); }
__device__ __forceinline__ void tmem_ld_wait() { tc5::wait_ld(); }

__device__ __forceinline__ float silu_mul(float g, float u) { return g / (1.0f + __expf(-g)) * u; }

// RMSNorm folded into the products around it.  The norm's weight is multiplied into the next matrix
// when the model is built, the activations are the bfloat16 copy of the raw residual, and what is left
// of the norm is one factor per token, applied to the float32 accumulator:
//   in_ssq   per token, `in_parts` partial sums of squares of the residual row this product reads;
//            factor = 1 / sqrt(sum(parts) * in_inv_k + eps).  Null: no factor.
//   out_ssq  (float32-add output only) after out += product, the partial sums of squares of the updated
//            rows, one per 128 output columns (ceil(N / 128) per token), and out_xhat, their bfloat16
//            copy [M, N] (row stride N): what the next product and its factor need.  Null: nothing.
// Sums are float32 and their order is fixed, so results do not depend on timing.
struct NormIO {
    const float* in_ssq;
    int in_parts;
    float in_inv_k;
    float eps;
    float* out_ssq;
    bf16* out_xhat;
};

// The q/k/v projection of an attention layer with what follows it fused into the epilogue (head size 128:
// one head per 128-row weight tile of the decode form, two per tile of the CTA-pair form): per-head RMSNorm of q and k with one shared weight
// each, rotation of pairs (i, i + 64) by the step's cos/sin tables, q to its buffer, k (normed, rotated)
// and v (raw) into the paged cache at the token's position.  Padding tokens (seq_of_token < 0) write
// nothing to the cache; k_pool == null writes no cache at all.
struct QkvIO {
    bf16* q_out;                 // [M, nq * 128]
    const float* qw;             // [128] or null: no norm
    const float* kw;
    float eps;
    const float* cosv;           // [M, 64]
    const float* sinv;
    const int* positions;        // [M]
    const int* seq_of_token;     // [M]
    const int* page_table;       // [sequences, max_pages]
    int max_pages;
    int page_size;
    bf16* k_pool;                // [pages, nkv, page_size, 128] of this layer
    bf16* v_pool;
    int nq;
    int nkv;
    int n_pages;                 // pages in the pools (the debug build checks every page id against it)
    int* status;                 // where the debug build records a page id or table index out of range (code 48)
};

// The q/k/v epilogue of a warp that holds one token's 128 sums of head `h` (all q heads, then the k heads, then
// the v heads), four per lane.  qkv_token_data() is what it reads from global memory beside the sums (the token's
// sequence, position and page, its rotation and the norm's weight); it depends on no sum and is asked for early.
struct QkvTok {
    int b, pos, page;
    float4 c4, s4, w4;
};
__device__ __forceinline__ QkvTok qkv_token_data(const QkvIO& qio, int gj, int h, int lane) {
    QkvTok t;
    t.b = -1; t.pos = 0; t.page = 0;
    t.c4 = make_float4(1.f, 1.f, 1.f, 1.f); t.s4 = make_float4(0.f, 0.f, 0.f, 0.f); t.w4 = make_float4(1.f, 1.f, 1.f, 1.f);
    const bool is_q = h < qio.nq, is_k = !is_q && h < qio.nq + qio.nkv;
    t.b = qio.seq_of_token[gj];
    if (!is_q && qio.k_pool != nullptr && t.b >= 0) {
        t.pos = qio.positions[gj];
        t.page = gg_page_w(qio.page_table + (size_t)t.b * qio.max_pages, t.pos / qio.page_size, qio.max_pages,
                           PageBounds{qio.n_pages, qio.status}, 48);
    }
    if (is_q || is_k) {
        const float* w = is_q ? qio.qw : qio.kw;
        if (w != nullptr) t.w4 = *reinterpret_cast<const float4*>(w + 4 * lane);
        const int i0 = 4 * (lane & 15);
        t.c4 = *reinterpret_cast<const float4*>(qio.cosv + (size_t)gj * 64 + i0);
        t.s4 = *reinterpret_cast<const float4*>(qio.sinv + (size_t)gj * 64 + i0);
    }
    return t;
}
// acc: features 4 lane .. 4 lane + 3 of head h of token gj, already multiplied by the folded norm's factor.
// Per-head RMSNorm and rotation for q and k; q to its buffer, k and v into the paged cache.  All 32 lanes call it.
__device__ __forceinline__ void qkv_token_finish(float4 acc, int gj, int h, int lane, const QkvIO& qio, const QkvTok& t) {
    const bool is_q = h < qio.nq, is_k = !is_q && h < qio.nq + qio.nkv;
    if (!is_q && (qio.k_pool == nullptr || t.b < 0)) return;
    float f[4] = {acc.x, acc.y, acc.z, acc.w};
    if (is_q || is_k) {
        if ((is_q ? qio.qw : qio.kw) != nullptr) {
            float ss = fmaf(f[0], f[0], fmaf(f[1], f[1], fmaf(f[2], f[2], f[3] * f[3])));
            ss = warp_sum(ss);
            const float scale = 1.0f / sqrtf(ss * (1.0f / 128.0f) + qio.eps);
            f[0] *= scale * t.w4.x; f[1] *= scale * t.w4.y; f[2] *= scale * t.w4.z; f[3] *= scale * t.w4.w;
        }
        const float cs[4] = {t.c4.x, t.c4.y, t.c4.z, t.c4.w}, sn[4] = {t.s4.x, t.s4.y, t.s4.z, t.s4.w};
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const float p = __shfl_xor_sync(0xffffffffu, f[u], 16);      // the other half of the pair
            f[u] = lane < 16 ? f[u] * cs[u] - p * sn[u] : p * sn[u] + f[u] * cs[u];
        }
    }
    bf16* dst;
    if (is_q) {
        dst = qio.q_out + ((size_t)gj * qio.nq + h) * 128;
    } else {
        if (t.page < 0) return;      // (debug build) outside the pools: nothing is written
        const int kvh = is_k ? h - qio.nq : h - qio.nq - qio.nkv;
        dst = (is_k ? qio.k_pool : qio.v_pool) +
              (((size_t)t.page * qio.nkv + kvh) * qio.page_size + (t.pos % qio.page_size)) * 128;
    }
    __nv_bfloat162 a = __floats2bfloat162_rn(f[0], f[1]), bb = __floats2bfloat162_rn(f[2], f[3]);
    *reinterpret_cast<uint2*>(dst + 4 * lane) = make_uint2(*reinterpret_cast<uint32_t*>(&a), *reinterpret_cast<uint32_t*>(&bb));
}

// One thread computes its token's factor (four running sums keep the loads independent).
__device__ __forceinline__ float norm_factor(const NormIO& nio, int token) {
    if (nio.in_ssq == nullptr) return 1.0f;
    const float* p = nio.in_ssq + (size_t)token * nio.in_parts;
    float t0 = 0.f, t1 = 0.f, t2 = 0.f, t3 = 0.f;
    int i = 0;
    for (; i + 4 <= nio.in_parts; i += 4) { t0 += p[i]; t1 += p[i + 1]; t2 += p[i + 2]; t3 += p[i + 3]; }
    for (; i < nio.in_parts; ++i) t0 += p[i];
    return 1.0f / sqrtf(((t0 + t1) + (t2 + t3)) * nio.in_inv_k + nio.eps);
}
// A whole warp computes one token's factor; every lane gets it.
__device__ __forceinline__ float norm_factor_warp(const NormIO& nio, int token, int lane) {
    if (nio.in_ssq == nullptr) return 1.0f;
    const float* p = nio.in_ssq + (size_t)token * nio.in_parts;
    float t = 0.f;
    for (int i = lane; i < nio.in_parts; i += 32) t += p[i];
    t = warp_sum(t);
    return 1.0f / sqrtf(t * nio.in_inv_k + nio.eps);
}

// Sixteen consecutive accumulator columns r[0..15] of output row gi, starting at column gj0 (a multiple
// of 16), already multiplied by the row's factor.  `ss` carries the sum of squares across a 128-column part.
__device__ __forceinline__ void store_row_chunk16(const uint32_t* r, int gi, int gj0, int N, void* __restrict__ out,
                                                  int out_mode, long long ldo, const NormIO& nio, float& ss) {
    const size_t o = (size_t)gi * ldo + gj0;
    const bool whole = gj0 + 16 <= N;
    if (out_mode == OUT_BF16) {
        bf16* op = (bf16*)out + o;
        if (whole && ((((uintptr_t)op) & 15) == 0)) {
            uint32_t pk[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                __nv_bfloat162 h2 = __floats2bfloat162_rn(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
                pk[j] = *reinterpret_cast<uint32_t*>(&h2);
            }
            reinterpret_cast<uint4*>(op)[0] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
            reinterpret_cast<uint4*>(op)[1] = make_uint4(pk[4], pk[5], pk[6], pk[7]);
        } else {
#pragma unroll
            for (int j = 0; j < 16; ++j)
                if (gj0 + j < N) op[j] = __float2bfloat16_rn(__uint_as_float(r[j]));
        }
        return;
    }
    float* op = (float*)out + o;
    const bool stats = nio.out_ssq != nullptr && out_mode == OUT_F32_ACC;
    bf16* xp = stats ? nio.out_xhat + (size_t)gi * N + gj0 : nullptr;
    if (whole && ((((uintptr_t)op) & 15) == 0) && (!stats || (((uintptr_t)xp) & 15) == 0)) {
        uint32_t pk[8];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float4 v = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                   __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
            float4* dst = reinterpret_cast<float4*>(op) + j;
            if (out_mode == OUT_F32_ACC) {
                const float4 old = *dst;
                v.x += old.x; v.y += old.y; v.z += old.z; v.w += old.w;
            }
            *dst = v;
            if (stats) {
                ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
                __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
                pk[2 * j] = *reinterpret_cast<uint32_t*>(&a);
                pk[2 * j + 1] = *reinterpret_cast<uint32_t*>(&b);
            }
        }
        if (stats) {
            reinterpret_cast<uint4*>(xp)[0] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
            reinterpret_cast<uint4*>(xp)[1] = make_uint4(pk[4], pk[5], pk[6], pk[7]);
        }
    } else {
#pragma unroll
        for (int j = 0; j < 16; ++j)
            if (gj0 + j < N) {
                float v = __uint_as_float(r[j]);
                if (out_mode == OUT_F32_ACC) v += op[j];
                op[j] = v;
                if (stats) { ss = fmaf(v, v, ss); xp[j] = __float2bfloat16_rn(v); }
            }
    }
    if (stats && (((gj0 & 127) == 112) || gj0 + 16 >= N)) {
        nio.out_ssq[(size_t)gi * ((N + 127) / 128) + (gj0 >> 7)] = ss;
        ss = 0.f;
    }
}

// Epilogue of the normal orientation for one thread: its row `gi` of the output, the 256 accumulator
// columns of tile column `tn` starting at tensor-memory address `taddr` (lane already selected).
// OUT_SWIGLU: the weight rows were interleaved in blocks of 64 gate rows and 64 up rows, so columns
// [0,64) and [128,192) of the tile are gates and the 64 columns after each are their ups; the output
// row has N / 2 columns.
__device__ __forceinline__ void epilogue_row_256(uint32_t taddr, int gi, int tn, int M, int N, void* __restrict__ out,
                                                 int out_mode, long long ldo, const NormIO& nio, float sc) {
    constexpr int BN = 256;
    if (out_mode == OUT_SWIGLU) {
#pragma unroll 1
        for (int cb = 0; cb < 2; ++cb) {
#pragma unroll 1
            for (int c0 = 0; c0 < 64; c0 += 16) {
                const int gcol = tn * BN + cb * 128 + c0;          // gate column in the interleaved product
                if (gcol >= N) return;
                uint32_t g[16], u[16];
                tmem_ld16(taddr + (uint32_t)(cb * 128 + c0), g);
                tmem_ld16(taddr + (uint32_t)(cb * 128 + 64 + c0), u);
                tmem_ld_wait();
                if (gi >= M) continue;
                const int ocol = (tn * 2 + cb) * 64 + c0;          // feature index
                bf16* op = (bf16*)out + (size_t)gi * ldo + ocol;
                const int nout = N / 2;
                if (ocol + 16 <= nout && ((((uintptr_t)op) & 15) == 0)) {
                    uint32_t pk[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        __nv_bfloat162 h2 = __floats2bfloat162_rn(
                            silu_mul(__uint_as_float(g[2 * j]) * sc, __uint_as_float(u[2 * j]) * sc),
                            silu_mul(__uint_as_float(g[2 * j + 1]) * sc, __uint_as_float(u[2 * j + 1]) * sc));
                        pk[j] = *reinterpret_cast<uint32_t*>(&h2);
                    }
                    reinterpret_cast<uint4*>(op)[0] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                    reinterpret_cast<uint4*>(op)[1] = make_uint4(pk[4], pk[5], pk[6], pk[7]);
                } else {
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        if (ocol + j < nout) op[j] = __float2bfloat16_rn(silu_mul(__uint_as_float(g[j]) * sc, __uint_as_float(u[j]) * sc));
                }
            }
        }
        return;
    }
    float ss = 0.f;          // running sum of squares of the updated row over 128 columns
    if (out_mode == OUT_F32_ACC && tn * BN + BN <= N && ((((uintptr_t)out) | ((uintptr_t)nio.out_xhat)) & 15) == 0 &&
        (ldo & 3) == 0 && (N & 7) == 0) {
        // Adding into the residual reads what is there: one thread's 16 columns at a time, every group would
        // wait a whole trip to L2 for its 64 bytes (about 20 us per tile, in the open after a product's last
        // tile).  So the old values of 64 columns are asked for at once, before the accumulator is read.
        const bool stats = nio.out_ssq != nullptr;
        const bool scaled = nio.in_ssq != nullptr;
        const bool live = gi < M;
        float* orow = (float*)out + (size_t)(live ? gi : 0) * ldo + tn * BN;
        bf16* xrow = stats ? nio.out_xhat + (size_t)(live ? gi : 0) * N + tn * BN : nullptr;
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 64) {
            float4 old[16];
            if (live) {
#pragma unroll
                for (int j = 0; j < 16; ++j) old[j] = reinterpret_cast<const float4*>(orow + c0)[j];
            }
            uint32_t r[64];
#pragma unroll
            for (int q = 0; q < 4; ++q) tmem_ld16(taddr + (uint32_t)(c0 + 16 * q), r + 16 * q);
            tmem_ld_wait();
            if (!live) continue;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                uint32_t pk[8];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float4 o = old[4 * q + j];
                    float4 v = make_float4(__uint_as_float(r[16 * q + 4 * j]), __uint_as_float(r[16 * q + 4 * j + 1]),
                                           __uint_as_float(r[16 * q + 4 * j + 2]), __uint_as_float(r[16 * q + 4 * j + 3]));
                    if (scaled) { v.x *= sc; v.y *= sc; v.z *= sc; v.w *= sc; }
                    v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
                    reinterpret_cast<float4*>(orow + c0 + 16 * q)[j] = v;
                    if (stats) {
                        ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
                        __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
                        pk[2 * j] = *reinterpret_cast<uint32_t*>(&a);
                        pk[2 * j + 1] = *reinterpret_cast<uint32_t*>(&b);
                    }
                }
                if (stats) {
                    reinterpret_cast<uint4*>(xrow + c0 + 16 * q)[0] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                    reinterpret_cast<uint4*>(xrow + c0 + 16 * q)[1] = make_uint4(pk[4], pk[5], pk[6], pk[7]);
                }
            }
            if (stats && (c0 & 64)) {            // a part of 128 columns is complete
                nio.out_ssq[(size_t)gi * ((N + 127) / 128) + ((tn * BN + c0) >> 7)] = ss;
                ss = 0.f;
            }
        }
        return;
    }
#pragma unroll 1
    for (int c0 = 0; c0 < BN; c0 += 16) {
        if (tn * BN + c0 >= N) break;
        uint32_t r[16];
        tmem_ld16(taddr + (uint32_t)c0, r);
        tmem_ld_wait();
        if (gi >= M) continue;
        if (nio.in_ssq != nullptr) {
#pragma unroll
            for (int j = 0; j < 16; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) * sc);
        }
        store_row_chunk16(r, gi, tn * BN + c0, N, out, out_mode, ldo, nio, ss);
    }
}

// Epilogue of the CTA-pair form for the q/k/v projection of a prefill step (head size 128): the tile's 256
// columns are heads 2 tn and 2 tn + 1 of token gi, all in this thread's row of tensor memory, so the per-head
// RMSNorm is a sum over the thread's own columns and the rotation's pairs (i, i + 64) need no exchange.  q
// goes to its buffer, k (normed, rotated) and v (raw) into the paged cache at the token's position, as in the
// decode form (QkvIO).  Every thread of the warp reads tensor memory; rows beyond M and tokens of padding
// write nothing.
__device__ __forceinline__ void epilogue_row_qkv(uint32_t taddr, int gi, int tn, int M, const QkvIO& qio, float sc) {
    const bool live = gi < M;
    const int nheads = qio.nq + 2 * qio.nkv;
    int b = -1, pos = 0, page = 0;
    if (live) {
        b = qio.seq_of_token[gi];
        if (qio.k_pool != nullptr && b >= 0) {
            pos = qio.positions[gi];
            page = gg_page_w(qio.page_table + (size_t)b * qio.max_pages, pos / qio.page_size, qio.max_pages,
                             PageBounds{qio.n_pages, qio.status}, 48);
            if (page < 0) b = -1;            // (debug build) outside the pools: this token writes no cache
        }
    }
    const float* cs = qio.cosv + (size_t)(live ? gi : 0) * 64;
    const float* sn = qio.sinv + (size_t)(live ? gi : 0) * 64;
#pragma unroll 1
    for (int hh = 0; hh < 2; ++hh) {
        const int h = tn * 2 + hh;
        if (h >= nheads) break;
        const bool is_q = h < qio.nq, is_k = !is_q && h < qio.nq + qio.nkv;
        const uint32_t tcol = taddr + (uint32_t)(hh * 128);
        bf16* dst = nullptr;
        if (live) {
            if (is_q) {
                dst = qio.q_out + ((size_t)gi * qio.nq + h) * 128;
            } else if (qio.k_pool != nullptr && b >= 0) {
                const int kvh = is_k ? h - qio.nq : h - qio.nq - qio.nkv;
                dst = (is_k ? qio.k_pool : qio.v_pool) +
                      (((size_t)page * qio.nkv + kvh) * qio.page_size + (pos % qio.page_size)) * 128;
            }
        }
        if (!is_q && !is_k) {                      // value head: the sums as they are
#pragma unroll 1
            for (int c = 0; c < 128; c += 16) {
                uint32_t r[16];
                tmem_ld16(tcol + (uint32_t)c, r);
                tmem_ld_wait();
                if (dst == nullptr) continue;
                uint32_t pk[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    __nv_bfloat162 h2 = __floats2bfloat162_rn(__uint_as_float(r[2 * j]) * sc, __uint_as_float(r[2 * j + 1]) * sc);
                    pk[j] = *reinterpret_cast<uint32_t*>(&h2);
                }
                reinterpret_cast<uint4*>(dst + c)[0] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                reinterpret_cast<uint4*>(dst + c)[1] = make_uint4(pk[4], pk[5], pk[6], pk[7]);
            }
            continue;
        }
        const float* w = is_q ? qio.qw : qio.kw;
        float scale = sc;
        if (w != nullptr) {
            float ss = 0.f;
#pragma unroll 1
            for (int c = 0; c < 128; c += 16) {
                uint32_t r[16];
                tmem_ld16(tcol + (uint32_t)c, r);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 16; ++j) { const float v = __uint_as_float(r[j]) * sc; ss = fmaf(v, v, ss); }
            }
            scale = sc * (1.0f / sqrtf(ss * (1.0f / 128.0f) + qio.eps));
        }
#pragma unroll 1
        for (int c = 0; c < 64; c += 16) {
            uint32_t lo[16], hi[16];
            tmem_ld16(tcol + (uint32_t)c, lo);
            tmem_ld16(tcol + (uint32_t)(64 + c), hi);
            tmem_ld_wait();
            if (dst == nullptr) continue;
            uint32_t pl[8], ph[8];
#pragma unroll
            for (int j4 = 0; j4 < 4; ++j4) {
                const float4 c4 = *reinterpret_cast<const float4*>(cs + c + 4 * j4);
                const float4 s4 = *reinterpret_cast<const float4*>(sn + c + 4 * j4);
                float4 wl = make_float4(1.f, 1.f, 1.f, 1.f), wh = wl;
                if (w != nullptr) {
                    wl = *reinterpret_cast<const float4*>(w + c + 4 * j4);
                    wh = *reinterpret_cast<const float4*>(w + 64 + c + 4 * j4);
                }
                const float cc[4] = {c4.x, c4.y, c4.z, c4.w}, sv[4] = {s4.x, s4.y, s4.z, s4.w};
                const float wlv[4] = {wl.x, wl.y, wl.z, wl.w}, whv[4] = {wh.x, wh.y, wh.z, wh.w};
                float ol[4], oh[4];
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                    const float x0 = __uint_as_float(lo[4 * j4 + t]) * scale * wlv[t];
                    const float x1 = __uint_as_float(hi[4 * j4 + t]) * scale * whv[t];
                    ol[t] = x0 * cc[t] - x1 * sv[t];
                    oh[t] = x1 * cc[t] + x0 * sv[t];
                }
                __nv_bfloat162 a = __floats2bfloat162_rn(ol[0], ol[1]), bb = __floats2bfloat162_rn(ol[2], ol[3]);
                pl[2 * j4] = *reinterpret_cast<uint32_t*>(&a); pl[2 * j4 + 1] = *reinterpret_cast<uint32_t*>(&bb);
                a = __floats2bfloat162_rn(oh[0], oh[1]); bb = __floats2bfloat162_rn(oh[2], oh[3]);
                ph[2 * j4] = *reinterpret_cast<uint32_t*>(&a); ph[2 * j4 + 1] = *reinterpret_cast<uint32_t*>(&bb);
            }
            reinterpret_cast<uint4*>(dst + c)[0] = make_uint4(pl[0], pl[1], pl[2], pl[3]);
            reinterpret_cast<uint4*>(dst + c)[1] = make_uint4(pl[4], pl[5], pl[6], pl[7]);
            reinterpret_cast<uint4*>(dst + 64 + c)[0] = make_uint4(ph[0], ph[1], ph[2], ph[3]);
            reinterpret_cast<uint4*>(dst + 64 + c)[1] = make_uint4(ph[4], ph[5], ph[6], ph[7]);
        }
    }
}

// The end of a decode-style epilogue: a warp holds one token's 128 consecutive accumulator columns
// [128 tile_a, 128 tile_a + 128), four per lane, already summed over the K splits and multiplied by the folded
// norm's factor, and applies the output mode (bf16 or float32 store, float32 add with the row statistics of the
// updated rows, or SwiGLU over interleaved gate/up blocks).  All 32 lanes call it.
// residual_prefetch() loads the four residual values at a lane's place ahead of time and says whether it did (the
// aligned path of finish_token_block, which then takes them as `old_pre` instead of loading them itself).
__device__ __forceinline__ bool residual_prefetch(int gj, int tile_a, int lane, void* out, int out_mode, long long ldo,
                                                  int N, const NormIO& nio, float4& old) {
    if (out_mode != OUT_F32_ACC) return false;
    const int gi0 = tile_a * BM + 4 * lane;
    if (gi0 + 4 > N) return false;
    const float* op = (const float*)out + (size_t)gj * ldo + gi0;
    const bool stats = nio.out_ssq != nullptr;
    if ((((uintptr_t)op) & 15) != 0 || (stats && (((uintptr_t)(nio.out_xhat + (size_t)gj * N + gi0)) & 7) != 0)) return false;
    old = *reinterpret_cast<const float4*>(op);
    return true;
}
__device__ __forceinline__ void finish_token_block(float4 acc, int gj, int tile_a, int lane, void* __restrict__ out,
                                                   int out_mode, long long ldo, int N, const NormIO& nio,
                                                   bool have_old = false, float4 old_pre = make_float4(0.f, 0.f, 0.f, 0.f)) {
    if (out_mode == OUT_SWIGLU) {
        // lanes 0..15 hold gates of 64 features, lanes 16..31 their ups
        const float ux = __shfl_down_sync(0xffffffffu, acc.x, 16), uy = __shfl_down_sync(0xffffffffu, acc.y, 16);
        const float uz = __shfl_down_sync(0xffffffffu, acc.z, 16), uw = __shfl_down_sync(0xffffffffu, acc.w, 16);
        const int feat = tile_a * 64 + 4 * lane;
        if (lane < 16 && feat < N / 2) {                 // N / 2 is a multiple of 64 here
            bf16* op = (bf16*)out + (size_t)gj * ldo + feat;
            __nv_bfloat162 a = __floats2bfloat162_rn(silu_mul(acc.x, ux), silu_mul(acc.y, uy));
            __nv_bfloat162 b = __floats2bfloat162_rn(silu_mul(acc.z, uz), silu_mul(acc.w, uw));
            if ((((uintptr_t)op) & 7) == 0) {
                *reinterpret_cast<uint2*>(op) = make_uint2(*reinterpret_cast<uint32_t*>(&a), *reinterpret_cast<uint32_t*>(&b));
            } else {
                op[0] = a.x; op[1] = a.y; op[2] = b.x; op[3] = b.y;
            }
        }
        return;
    }
    const int gi0 = tile_a * BM + 4 * lane;              // first of this lane's four features
    const bool stats = nio.out_ssq != nullptr && out_mode == OUT_F32_ACC;
    float ss = 0.f;
    if (gi0 < N) {
        const bool whole = gi0 + 4 <= N;
        const size_t o = (size_t)gj * ldo + gi0;
        float f[4] = {acc.x, acc.y, acc.z, acc.w};
        if (out_mode == OUT_BF16) {
            bf16* op = (bf16*)out + o;
            if (whole && (((uintptr_t)op) & 7) == 0) {
                __nv_bfloat162 a = __floats2bfloat162_rn(f[0], f[1]), b = __floats2bfloat162_rn(f[2], f[3]);
                *reinterpret_cast<uint2*>(op) = make_uint2(*reinterpret_cast<uint32_t*>(&a), *reinterpret_cast<uint32_t*>(&b));
            } else {
#pragma unroll
                for (int t = 0; t < 4; ++t)
                    if (gi0 + t < N) op[t] = __float2bfloat16_rn(f[t]);
            }
        } else {
            float* op = (float*)out + o;
            bf16* xp = stats ? nio.out_xhat + (size_t)gj * N + gi0 : nullptr;
            if (whole && (((uintptr_t)op) & 15) == 0 && (!stats || (((uintptr_t)xp) & 7) == 0)) {
                float4 w4 = make_float4(f[0], f[1], f[2], f[3]);
                if (out_mode == OUT_F32_ACC) {
                    const float4 old = have_old ? old_pre : *reinterpret_cast<float4*>(op);
                    w4.x += old.x; w4.y += old.y; w4.z += old.z; w4.w += old.w;
                }
                *reinterpret_cast<float4*>(op) = w4;
                if (stats) {
                    ss = fmaf(w4.x, w4.x, ss); ss = fmaf(w4.y, w4.y, ss); ss = fmaf(w4.z, w4.z, ss); ss = fmaf(w4.w, w4.w, ss);
                    __nv_bfloat162 a = __floats2bfloat162_rn(w4.x, w4.y), b = __floats2bfloat162_rn(w4.z, w4.w);
                    *reinterpret_cast<uint2*>(xp) = make_uint2(*reinterpret_cast<uint32_t*>(&a), *reinterpret_cast<uint32_t*>(&b));
                }
            } else {
#pragma unroll
                for (int t = 0; t < 4; ++t)
                    if (gi0 + t < N) {
                        float val = f[t];
                        if (out_mode == OUT_F32_ACC) val += op[t];
                        op[t] = val;
                        if (stats) { ss = fmaf(val, val, ss); xp[t] = __float2bfloat16_rn(val); }
                    }
            }
        }
    }
    if (stats) {
        ss = warp_sum(ss);                               // one 128-feature part per tile
        if (lane == 0) nio.out_ssq[(size_t)gj * ((N + 127) / 128) + tile_a] = ss;
    }
}

template <int BN> constexpr int tmem_cols() { return BN < 32 ? 32 : BN; }

__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float4 ld_cluster_f32x4(uint32_t local_addr, uint32_t rank) {
    uint32_t remote;
    float4 v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(remote) : "memory");
    return v;
}


// A row of four floats into the shared memory of CTA `rank` of the cluster, completing 16 bytes of the transaction
// count of that CTA's mbarrier `bar_local_addr` (same offset in every CTA) once the store is visible there.
__device__ __forceinline__ void st_async_f32x4(uint32_t local_addr, uint32_t bar_local_addr, uint32_t rank, float4 v) {
    uint32_t remote, rbar;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(rbar) : "r"(bar_local_addr), "r"(rank));
    asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.f32 [%0], {%1, %2, %3, %4}, [%5];"
                 ::"r"(remote), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w), "r"(rbar) : "memory");
}
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }

constexpr int MAX_CLUSTER = 8;
// The 16-token decode form keeps a receive area of its own beside the pipeline stages: RECV16_SLOTS rows of 128
// floats, enough for [source rank][owner's token] with up to 8 ranks (S * ceil(16 / S) <= 21).
constexpr int RECV16_SLOTS = 22;
template <int BN, bool SWAP> constexpr int recv_bytes() { return (SWAP && BN == 16) ? RECV16_SLOTS * BM * 4 : 0; }

// cluster_reduce != 0: the grid was launched with clusters of gridDim.z CTAs along z (the K splits).
template <int BN, int STAGES, bool SWAP, int MINB>
__global__ void __launch_bounds__(NUM_THREADS, MINB) gemm_tc_kernel(
    const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
    void* __restrict__ out, int out_mode, long long ldo, int M, int N, int K, int kb_per_split,
    float* __restrict__ partial, int cluster_reduce, int* __restrict__ status, const NormIO nio, const QkvIO qio) {
    constexpr int B_BYTES = BN * BK * 2;
    constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* full = (uint64_t*)(smem + STAGES * STAGE_BYTES);
    uint64_t* empty = full + STAGES;
    uint64_t* accum = empty + STAGES;
    uint64_t* recv_bar = accum + 1;
    // the tile goes through shared memory when K splits are added inside the cluster, for the fused
    // activation, and (decode form) whenever a norm is folded into this product
    // (only the decode form splits K or fuses the activation; the launcher sees to that)
    const bool staged = SWAP && (cluster_reduce || out_mode == OUT_SWIGLU || out_mode == OUT_QKV ||
                                 (partial == nullptr && (nio.in_ssq != nullptr || nio.out_ssq != nullptr)));
    uint32_t* tmem_slot = (uint32_t*)(recv_bar + 1);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
    // decode form with a folded norm: the factor of every token of the tile, computed by the epilogue warps while
    // the weights still stream (inside the barrier area for 16 tokens, behind it otherwise)
    float* sfac = reinterpret_cast<float*>(smem + STAGES * STAGE_BYTES + (BN <= 16 ? 128 : 256));
    // Up to 16 tokens the K splits of a cluster are added without any barrier at the end: every CTA sends the
    // partial rows of token j to the CTA that owns it (rank j mod S) with st.async into a receive area that is
    // not part of the pipeline stages, each row completing 512 bytes of the owner's mbarrier; the owner waits
    // for the bytes it expects and adds them in rank order.  The one cluster barrier that is left says "my
    // mbarrier is initialised": its arriving half is in the prologue, its waiting half right before the first
    // row is sent, by which time it has long completed.  (Both end-of-kernel barriers and the exchange between
    // them cost 6 % of a decode step at batch 1 and 8, measured by compiling them out.)
    // At 32 tokens the receive area lies in the pipeline stages behind the CTA's own tile, so the barrier has
    // to say "my stages are free" as well: there its arriving half is executed by every thread as soon as
    // this CTA's last MMA has completed (`push3`; 12 layers at batch 32: 1.769 -> 1.754 ms).  From 64 tokens on
    // the owner pulls, with a barrier before and one after: the same scheme measured slower there (batch 64:
    // 2.404 -> 2.423 ms), and at 128 tokens tile and receive area would not fit the stages.
    constexpr bool HAS_RECV = recv_bytes<BN, SWAP>() > 0;
    const bool push2 = HAS_RECV && staged && cluster_reduce != 0;
    const bool push3 = !HAS_RECV && SWAP && BN == 32 && staged && cluster_reduce != 0;
    uint8_t* recv2 = HAS_RECV ? smem + STAGES * STAGE_BYTES + 256 : smem + (size_t)BN * BM * 4;

    pdl_launch();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile_a = blockIdx.x, tile_b = blockIdx.y, split = blockIdx.z;
    const int num_kb = (K + BK - 1) / BK;
    const int kb0 = split * kb_per_split;
    const int nkb = min(num_kb, kb0 + kb_per_split) - kb0;   // >= 1 by construction of the grid

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        mbar_init(accum, 1);
        mbar_init(recv_bar, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tmA) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tmB) : "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(tmem_slot)), "r"(tmem_cols<BN>()) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // tokens of this tile that this CTA adds up when the splits are pushed: j with j mod S == split
    int n_owned = 0;
    if (push2 || push3) {
        const int S = (int)gridDim.z, cols = min(BN, M - tile_b * BN);
        n_owned = split < cols ? (cols - split + S - 1) / S : 0;
        if (threadIdx.x == 0 && n_owned > 0) mbar_expect_tx(recv_bar, (uint32_t)(S * n_owned * BM * 4));
        if (push2) cluster_arrive();
    }

    if (warp == 0) {
        if (lane == 0) {
            // The weights are written by no kernel: their first tiles stream in while the kernel before
            // this one is still finishing.  The activations are that kernel's output and wait for it.
            const int pre = nkb < STAGES ? nkb : STAGES;
            for (int i = 0; i < pre; ++i) {
                mbar_expect_tx(&full[i], STAGE_BYTES);
                uint8_t* sa = smem + i * STAGE_BYTES;
                if (SWAP) tma_load_2d(sa, &tmA, &full[i], (kb0 + i) * BK, tile_a * BM);
                else tma_load_2d(sa + A_BYTES, &tmB, &full[i], (kb0 + i) * BK, tile_b * BN);
            }
            pdl_wait();
            for (int i = 0; i < pre; ++i) {
                uint8_t* sa = smem + i * STAGE_BYTES;
                if (SWAP) tma_load_2d(sa + A_BYTES, &tmB, &full[i], (kb0 + i) * BK, tile_b * BN);
                else tma_load_2d(sa, &tmA, &full[i], (kb0 + i) * BK, tile_a * BM);
            }
            for (int i = pre; i < nkb; ++i) {
                const int s = i % STAGES;
                const uint32_t ph = (uint32_t)(i / STAGES) & 1u;
                if (!mbar_wait(&empty[s], ph ^ 1u, abort_flag, status, 1)) break;
                mbar_expect_tx(&full[s], STAGE_BYTES);
                uint8_t* sa = smem + s * STAGE_BYTES;
                tma_load_2d(sa, &tmA, &full[s], (kb0 + i) * BK, tile_a * BM);
                tma_load_2d(sa + A_BYTES, &tmB, &full[s], (kb0 + i) * BK, tile_b * BN);
            }
        }
        if (push3) {
            __syncwarp();
            mbar_wait(accum, 0, abort_flag, status, 1);       // the last MMA has read the stages
            cluster_arrive();
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = make_idesc(BM, BN);
            bool ok = true;
            for (int i = 0; i < nkb && ok; ++i) {
                const int s = i % STAGES;
                const uint32_t ph = (uint32_t)(i / STAGES) & 1u;
                ok = mbar_wait(&full[s], ph, abort_flag, status, 2);
                if (!ok) break;
                tc_fence_after();
                const uint32_t sa = smem_u32(smem + s * STAGE_BYTES);
                const uint64_t adesc = make_smem_desc(sa);
                const uint64_t bdesc = make_smem_desc(sa + A_BYTES);
#pragma unroll
                for (int k = 0; k < BK / UMMA_K; ++k) {
                    // advance 32 bytes (16 bf16) along K inside the swizzle atom: +2 in 16-byte units
                    umma(tmem_base, adesc + 2 * k, bdesc + 2 * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
                }
                umma_commit(&empty[s]);
            }
            if (ok) umma_commit(accum);
        }
        if (push3) {
            __syncwarp();
            mbar_wait(accum, 0, abort_flag, status, 2);
            cluster_arrive();
        }
    } else {
        // epilogue: warp w reads tensor-memory lanes 32*(w%4) .. +31 (row i of D is lane i)
        const int q = warp & 3;
        const int row = q * 32 + lane;           // row of the D tile held by this thread
        const int gi = tile_a * BM + row;        // global row of D (A side)
        const int RA = SWAP ? N : M, RB = SWAP ? M : N;
        pdl_wait();                              // the output may still be in use by earlier kernels
        const float sc = (!SWAP && gi < RA) ? norm_factor(nio, gi) : 1.0f;
        if (SWAP && staged && nio.in_ssq != nullptr) {
            const int t = (int)threadIdx.x - 64;             // the epilogue warps are threads 64 .. 191
            if (t < BN && tile_b * BN + t < M) sfac[t] = norm_factor(nio, tile_b * BN + t);
        }
        mbar_wait(accum, 0, abort_flag, status, 3);
        if (push3) cluster_arrive();             // the tile is complete in tensor memory: the stages are free from here
        if (!*abort_flag) {
            tc_fence_after();
            float ss = 0.f;
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 16) {
                if (tile_b * BN + c0 >= RB) break;          // whole warp agrees: columns beyond the extent
                uint32_t r[16];
                tmem_ld16(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)c0, r);
                tmem_ld_wait();
                if (staged) {
                    // own partial sums to own shared memory, [column][row]: the pipeline stages are free now
                    float* stage = reinterpret_cast<float*>(smem);
#pragma unroll
                    for (int j = 0; j < 16; ++j) stage[(c0 + j) * BM + row] = __uint_as_float(r[j]);
                    continue;
                }
                if (gi >= RA) continue;
                const int gj0 = tile_b * BN + c0;
                if (partial != nullptr) {
                    float* p = partial + (size_t)split * M * N;
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int gj = gj0 + j;
                        if (gj < RB) {
                            if (SWAP) p[(size_t)gj * N + gi] = __uint_as_float(r[j]);
                            else p[(size_t)gi * N + gj] = __uint_as_float(r[j]);
                        }
                    }
                } else if (SWAP) {
                    // out[m = gj][n = gi]: for a fixed j the 32 lanes write 32 consecutive n
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int gj = gj0 + j;
                        if (gj < RB) {
                            const float v = __uint_as_float(r[j]);
                            const size_t o = (size_t)gj * ldo + gi;
                            if (out_mode == OUT_BF16) ((bf16*)out)[o] = __float2bfloat16_rn(v);
                            else if (out_mode == OUT_F32) ((float*)out)[o] = v;
                            else ((float*)out)[o] += v;
                        }
                    }
                } else {
                    // out[m = gi][n = gj0 .. gj0+15]: 16 consecutive n per thread
                    if (nio.in_ssq != nullptr) {
#pragma unroll
                        for (int j = 0; j < 16; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) * sc);
                    }
                    store_row_chunk16(r, gi, gj0, N, out, out_mode, ldo, nio, ss);
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (staged) {
        // Every CTA of the cluster passes its barriers exactly once each, whatever happened before.
        const bool pull_reduce = cluster_reduce && !push2 && !push3;
        if (pull_reduce) cluster_arrive();       // (waited for below, after the loads that do not need the other ranks)
        // Decode form: a warp per token.  Each lane adds four consecutive features of the 128 of this tile over
        // the cluster's ranks, in rank order, then the epilogue of the output mode.  Up to 32 tokens per tile
        // the partial sums are *pushed* to the CTA that owns the token (rank j mod S) and the owner adds what it
        // received from its own shared memory: remote stores need no round trip (measured: 9.1 -> 8.6 us for the
        // O product at 8 tokens).  At 16 tokens the rows go out with st.async and no cluster barrier is left at
        // the end of the kernel (see `push2` above); at 32 tokens the receive area lies in the pipeline stages,
        // so the one barrier also says that they are free (`push3`).  With 64 tokens per tile the exchange is
        // bound by its volume, not its latency, and pushing was slower than pulling in either form, so from
        // there on the owner pulls.
        const int S = cluster_reduce ? (int)gridDim.z : 1;
        const int cols = min(BN, M - tile_b * BN);
        const uint32_t stage = smem_u32(smem);
        constexpr int WARPS = NUM_THREADS / 32;
        const bool push = push2 || push3;
        const int LJ = (cols + S - 1) / S;                           // tokens an owner handles at most
        // where the pushed rows land, [source rank][owner's token][128] float32: beside the stages (16 tokens) or
        // behind the tile in them (32 tokens)
        const uint32_t recv = smem_u32(recv2);
        const uint8_t* recv_mine = recv2;
        if (push) {
            cluster_wait();              // every CTA of the cluster has initialised its mbarrier (and freed its stages)
            if (!*abort_flag) {
                for (int j = warp; j < cols; j += WARPS) {
                    const float4 v = *reinterpret_cast<const float4*>(smem + (size_t)(j * BM + 4 * lane) * 4);
                    st_async_f32x4(recv + 4u * (uint32_t)((split * LJ + j / S) * BM + 4 * lane), smem_u32(recv_bar),
                                   (uint32_t)(j % S), v);
                }
            }
        }
        // The residual values of this warp's first rounds are asked for before the wait for the other ranks (a
        // round is one token per warp; a pulling owner has cols / S tokens on six warps).
        const int j_first = push ? warp * S + split : split * WARPS + warp;
        constexpr int RPRE = 3;
        float4 old_r[RPRE];
        bool have_r[RPRE];
#pragma unroll
        for (int r = 0; r < RPRE; ++r) {
            const int j = j_first + r * S * WARPS;
            old_r[r] = make_float4(0.f, 0.f, 0.f, 0.f);
            have_r[r] = SWAP && !push && out_mode != OUT_QKV && j < cols &&
                        residual_prefetch(tile_b * BN + j, tile_a, lane, out, out_mode, ldo, N, nio, old_r[r]);
        }
        if (pull_reduce) cluster_wait();
        // An owner that pulls from at most four ranks asks for the rows of several of its tokens at once (a gate-up
        // product of 64 tokens has 32 tokens per owner, five to six per warp: one round trip through the cluster
        // per token would stand in the open six times).
        // A pulling owner says "I have read what I need from your shared memory" as soon as the rows of its last
        // tokens are in its registers, and waits for the others to say so after its last epilogue: the last
        // global stores run beside the barrier instead of before it.
        bool left = !(cluster_reduce && !push);       // no closing barrier in the other forms
        auto pull_grouped = [&](auto uc) {
            constexpr int U = decltype(uc)::value, SP = MAX_CLUSTER / U;
            const int stride = S * WARPS;
            int round = 0;
            for (int j0 = j_first; j0 < cols; j0 += U * stride, round += U) {
                float4 v[U][SP];
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const int j = j0 + u * stride;
#pragma unroll
                    for (int qq = 0; qq < SP; ++qq)
                        v[u][qq] = (qq < S && j < cols) ? ld_cluster_f32x4(stage + 4u * (uint32_t)(j * BM + 4 * lane), qq)
                                                        : make_float4(0.f, 0.f, 0.f, 0.f);
                }
                float4 accs[U];
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    accs[u] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                    for (int qq = 0; qq < SP; ++qq) { accs[u].x += v[u][qq].x; accs[u].y += v[u][qq].y; accs[u].z += v[u][qq].z; accs[u].w += v[u][qq].w; }
                }
                if (!left && j0 + U * stride >= cols) { cluster_arrive(); left = true; }
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const int j = j0 + u * stride, r = round + u;
                    if (j >= cols) break;
                    const int gj = tile_b * BN + j;
                    float4 acc = accs[u];
                    if (nio.in_ssq != nullptr) { const float sc = sfac[j]; acc.x *= sc; acc.y *= sc; acc.z *= sc; acc.w *= sc; }
                    float4 old4 = r == 0 ? old_r[0] : (r == 1 ? old_r[1] : old_r[2]);
                    bool have_old = r < RPRE && (r == 0 ? have_r[0] : (r == 1 ? have_r[1] : have_r[2]));
                    if (r >= RPRE) have_old = residual_prefetch(gj, tile_a, lane, out, out_mode, ldo, N, nio, old4);
                    finish_token_block(acc, gj, tile_a, lane, out, out_mode, ldo, N, nio, have_old, old4);
                }
            }
        };
        // (only the forms that pull: up to 32 tokens the rows are pushed)
        const bool grouped = SWAP && BN >= 64 && !push && out_mode != OUT_QKV && S <= 4 && !*abort_flag;
        if constexpr (SWAP && BN >= 64) {
            if (grouped) {
                if (S <= 2) pull_grouped(std::integral_constant<int, 4>{});
                else pull_grouped(std::integral_constant<int, 2>{});
            }
        }
        if (!*abort_flag && SWAP && !grouped) {
            bool received = !push;           // pushed rows: the wait comes after everything that does not need them
            int round = 0;
            for (int j = j_first; j < cols; j += S * WARPS, ++round) {
                const int gj = tile_b * BN + j;                      // token
                // What the epilogue reads from global memory does not depend on the sums: the folded norm's
                // factor, the residual values, for q/k/v the token's sequence, position, page and rotation.  All of
                // it is asked for here, before the wait for the other ranks' rows, so that its latency (two to
                // three dependent loads for q/k/v) runs beside the exchange instead of behind it.
                const float sc = nio.in_ssq != nullptr ? sfac[j] : 1.0f;
                float4 old4 = round == 0 ? old_r[0] : (round == 1 ? old_r[1] : old_r[2]);
                bool have_old = round < RPRE && (round == 0 ? have_r[0] : (round == 1 ? have_r[1] : have_r[2]));
                if (!have_old && out_mode != OUT_QKV && (push || round >= RPRE))
                    have_old = residual_prefetch(gj, tile_a, lane, out, out_mode, ldo, N, nio, old4);
                QkvTok qt;
                if (out_mode == OUT_QKV) qt = qkv_token_data(qio, gj, tile_a, lane);       // this tile is head `tile_a`
                if (!received) {
                    if (!mbar_wait(recv_bar, 0, abort_flag, status, 5)) break;
                    received = true;
                }
                float4 v[MAX_CLUSTER];
                if (push) {
                    const uint8_t* mine = recv_mine + (size_t)((j / S) * BM + 4 * lane) * 4;
#pragma unroll
                    for (int qq = 0; qq < MAX_CLUSTER; ++qq)
                        v[qq] = qq < S ? *reinterpret_cast<const float4*>(mine + (size_t)qq * LJ * BM * 4)
                                       : make_float4(0.f, 0.f, 0.f, 0.f);
                } else {
#pragma unroll
                    for (int qq = 0; qq < MAX_CLUSTER; ++qq)
                        v[qq] = qq < S ? ld_cluster_f32x4(stage + 4u * (uint32_t)(j * BM + 4 * lane), qq)
                                       : make_float4(0.f, 0.f, 0.f, 0.f);
                }
                float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int qq = 0; qq < MAX_CLUSTER; ++qq) { acc.x += v[qq].x; acc.y += v[qq].y; acc.z += v[qq].z; acc.w += v[qq].w; }
                if (!left && j + S * WARPS >= cols) { cluster_arrive(); left = true; }
                if (nio.in_ssq != nullptr) { acc.x *= sc; acc.y *= sc; acc.z *= sc; acc.w *= sc; }
                if (out_mode == OUT_QKV) {
                    qkv_token_finish(acc, gj, tile_a, lane, qio, qt);
                    continue;
                }
                finish_token_block(acc, gj, tile_a, lane, out, out_mode, ldo, N, nio, have_old, old4);
            }
        }
        if (cluster_reduce && !push) {
            if (!left) cluster_arrive();          // (a warp without a token, or a kernel that gave up)
            cluster_wait();                       // nobody leaves while its shared memory may still be read
        }
    }
    if (*abort_flag) {
        // a wait ran out: give copies and instructions in flight time to land before the memory goes away
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000LL) { }
        __syncthreads();
    }
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols<BN>()) : "memory");
    }
}

// out[m, n] = epilogue( sum over splits of partial[s, m, n] ), splits added in index order.
__global__ void splitk_reduce_kernel(const float* partial, void* __restrict__ out, int out_mode,
                                     long long ldo, int M, int N, int splits) {
    pdl_launch();
    pdl_wait();
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long total = (long long)M * N;
    if (idx >= total) return;
    const int m = (int)(idx / N), n = (int)(idx - (long long)m * N);
    float s = 0.f;
    for (int k = 0; k < splits; ++k) s += partial[(size_t)k * total + idx];
    const size_t o = (size_t)m * ldo + n;
    if (out_mode == OUT_BF16) ((bf16*)out)[o] = __float2bfloat16_rn(s);
    else if (out_mode == OUT_F32) ((float*)out)[o] = s;
    else ((float*)out)[o] += s;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (fn == nullptr) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}

// A [rows, K] bf16 matrix with row stride ld (elements), boxes of [box_rows x 64], 128-byte swizzle.
int make_map(CUtensorMap* map, const void* ptr, int rows, int K, long long ld, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (fn == nullptr) return GG_ERR_TMAP;
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : GG_ERR_TMAP;
}

// ------------------------------------------------------------------------------------------- prefill form, persistent
// One CTA per SM walks over output tiles of 128 x 256 (token rows fastest, so the CTAs that run
// together share weight tiles in L2).  The shared-memory ring runs on across tile boundaries, and the
// accumulator is double buffered in tensor memory (2 x 256 columns): while the four epilogue warps
// drain tile i, the MMA thread already accumulates tile i + 1.
template <int STAGES>
__global__ void __launch_bounds__(NUM_THREADS, 1) gemm_tc_persistent_kernel(
    const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
    void* __restrict__ out, int out_mode, long long ldo, int M, int N, int K, int* __restrict__ status,
    const NormIO nio) {
    constexpr int BN = 256;
    constexpr int B_BYTES = BN * BK * 2;
    constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* full = (uint64_t*)(smem + STAGES * STAGE_BYTES);
    uint64_t* empty = full + STAGES;
    uint64_t* acc_full = empty + STAGES;       // [2]
    uint64_t* acc_empty = acc_full + 2;        // [2]
    uint32_t* tmem_slot = (uint32_t*)(acc_empty + 2);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

    pdl_launch();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int num_kb = (K + BK - 1) / BK;
    const int tiles_m = (M + BM - 1) / BM, tiles_n = (N + BN - 1) / BN;
    const int total = tiles_m * tiles_n;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 128); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tmA) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tmB) : "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(tmem_slot)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            int it = 0;
            bool first = true, ok = true;
            for (int t = blockIdx.x; t < total && ok; t += gridDim.x) {
                const int tm = t % tiles_m, tn = t / tiles_m;
                int kb = 0;
                if (first) {
                    // weights of the first tile before the dependency wait (see the decode form)
                    const int pre = num_kb < STAGES ? num_kb : STAGES;
                    for (int i = 0; i < pre; ++i) {
                        mbar_expect_tx(&full[i], STAGE_BYTES);
                        tma_load_2d(smem + i * STAGE_BYTES + A_BYTES, &tmB, &full[i], i * BK, tn * BN);
                    }
                    pdl_wait();
                    for (int i = 0; i < pre; ++i) tma_load_2d(smem + i * STAGE_BYTES, &tmA, &full[i], i * BK, tm * BM);
                    kb = pre;
                    it = pre;
                    first = false;
                }
                for (; kb < num_kb; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (uint32_t)(it / STAGES) & 1u;
                    if (!mbar_wait(&empty[s], ph ^ 1u, abort_flag, status, 1)) { ok = false; break; }
                    mbar_expect_tx(&full[s], STAGE_BYTES);
                    uint8_t* sa = smem + s * STAGE_BYTES;
                    tma_load_2d(sa, &tmA, &full[s], kb * BK, tm * BM);
                    tma_load_2d(sa + A_BYTES, &tmB, &full[s], kb * BK, tn * BN);
                }
            }
            if (first) pdl_wait();
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = make_idesc(BM, BN);
            int it = 0, i = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < total && ok; t += gridDim.x, ++i) {
                const int buf = i & 1;
                const uint32_t aph = (uint32_t)(i >> 1) & 1u;
                ok = mbar_wait(&acc_empty[buf], aph ^ 1u, abort_flag, status, 4);     // the epilogue has drained it
                if (!ok) break;
                tc_fence_after();
                const uint32_t tacc = tmem_base + (uint32_t)(buf * BN);
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (uint32_t)(it / STAGES) & 1u;
                    ok = mbar_wait(&full[s], ph, abort_flag, status, 2);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t sa = smem_u32(smem + s * STAGE_BYTES);
                    const uint64_t adesc = make_smem_desc(sa);
                    const uint64_t bdesc = make_smem_desc(sa + A_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)
                        umma(tacc, adesc + 2 * k, bdesc + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    umma_commit(&empty[s]);
                }
                if (ok) umma_commit(&acc_full[buf]);
            }
        }
    } else {
        const int q = warp & 3;
        const int row = q * 32 + lane;
        pdl_wait();
        int i = 0;
        for (int t = blockIdx.x; t < total; t += gridDim.x, ++i) {
            const int tm = t % tiles_m, tn = t / tiles_m;
            const int buf = i & 1;
            const uint32_t aph = (uint32_t)(i >> 1) & 1u;
            const int gi = tm * BM + row;
            const float sc = gi < M ? norm_factor(nio, gi) : 1.0f;      // while the tile is still being multiplied
            if (!mbar_wait(&acc_full[buf], aph, abort_flag, status, 3)) break;
            tc_fence_after();
            epilogue_row_256(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * BN), gi, tn, M, N, out, out_mode, ldo, nio, sc);
            tc_fence_before();
            mbar_arrive(&acc_empty[buf]);        // 128 arrivals free the accumulator for tile i + 2
        }
    }

    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000LL) { }
        __syncthreads();
    }
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
    }
}

int launch_persistent(const CUtensorMap& ta, const CUtensorMap& tb, void* out, int out_mode, long long ldo, int M, int N,
                      int K, int* status, const NormIO& nio, cudaStream_t stream) {
    constexpr int STAGES = 4;
    constexpr int smem = STAGES * (A_BYTES + 256 * BK * 2) + 1024 + 256;
    static int sms = 0;
    auto kern = gemm_tc_persistent_kernel<STAGES>;
    if (sms == 0) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return (int)e;
        int dev = 0, n = 0;
        if ((e = cudaGetDevice(&dev)) != cudaSuccess) return (int)e;
        if ((e = cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return (int)e;
        sms = n > 0 ? n : 148;
    }
    const int total = ((M + BM - 1) / BM) * ((N + 255) / 256);
    const int grid = total < sms ? total : sms;
    return gg_launch(kern, dim3(grid), dim3(NUM_THREADS), smem, stream, 1, ta, tb, out, out_mode, ldo, M, N, K, status, nio);
}

// ------------------------------------------------------------------------------------------- prefill form, CTA pairs
// Two CTAs of a cluster work on one 256 x 256 output tile with tcgen05.mma.cta_group::2: each CTA
// stages its own 128 rows of A and its own 128 of the 256 B rows, the leader CTA issues the MMAs
// for both, and each CTA ends up with its 128 rows of the tile in its own tensor memory.  Per CTA
// and 64-wide K slab that is 32 KB of operands for 128 x 256 x 64 multiply-adds instead of 48 KB,
// so six stages fit in shared memory and cover the L2 latency that four 48 KB stages do not
// (the single-CTA form leaves the tensor pipe idle 22 % of the time).  Persistent over tiles, with
// the accumulator double buffered as in gemm_tc_persistent_kernel.
//
// Barriers live at the same shared-memory offsets in both CTAs.  full[s]: in the leader; it expects
// the bytes of both CTAs' copies (the peer's TMA signals the leader's barrier).  empty[s] and
// acc_full[b]: in both; the leader's tcgen05.commit arrives on both at once.  acc_empty[b]: in the
// leader; the 128 epilogue threads of each CTA arrive on it, the peer's through the cluster.
constexpr uint32_t PEER_BIT_MASK = 0xFEFFFFFFu;

__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar) & PEER_BIT_MASK), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void umma_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc) : "memory");
}
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
    const uint16_t mask = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(smem_u32(bar)), "h"(mask) : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint64_t* bar, uint32_t rank) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(bar)), "r"(rank));
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(remote) : "memory");
}

template <int STAGES>
__global__ void __launch_bounds__(NUM_THREADS, 1) gemm_tc_pair_kernel(
    const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
    void* __restrict__ out, int out_mode, long long ldo, int M, int N, int K, int* __restrict__ status,
    const NormIO nio, int splits, int whole, int kb_per_split, float* __restrict__ partial, const QkvIO qio) {
    constexpr int BN = 256;                     // columns of the pair's tile (each CTA stages 128 of the B rows)
    constexpr int HALF_B_BYTES = 128 * BK * 2;
    constexpr int STAGE_BYTES = A_BYTES + HALF_B_BYTES;      // per CTA: 32 KB
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* full = (uint64_t*)(smem + STAGES * STAGE_BYTES);
    uint64_t* empty = full + STAGES;
    uint64_t* acc_full = empty + STAGES;
    uint64_t* acc_empty = acc_full + 2;
    uint32_t* tmem_slot = (uint32_t*)(acc_empty + 2);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

    pdl_launch();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    uint32_t rank;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
    const bool leader = rank == 0;
    const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
    const int num_kb = (K + BK - 1) / BK;
    const int tiles_m = (M + 255) / 256, tiles_n = (N + BN - 1) / BN;
    // With few tiles (prompts of a few hundred tokens) the K range of a tile is split over `splits` work items,
    // so that all pairs have work.  The first `whole` tiles (in tile order, a multiple of tiles_m: whole tile
    // columns) are not split: the waves that the tiles fill anyway; the rest, a last wave that would be nearly
    // empty, or all of them, are.  The items of a split tile leave float32 partial tiles in `partial`
    // [splits][M][columns from the first split tile column on] and gemm_splitk_finish_kernel adds them and
    // applies the output mode.
    const int tiles = tiles_m * tiles_n;
    const int total = whole + (tiles - whole) * splits;
    const int tn_split = whole / tiles_m;                       // first tile column that is split
    const int NS = N - tn_split * BN;                           // columns of the partial tiles
    // work item t -> (tile, split, is it one of a split tile's)
    auto item_of = [&](int t, int& tile, int& split, bool& parted) {
        if (t < whole) { tile = t; split = 0; parted = false; }
        else { const int u = t - whole; tile = whole + u / splits; split = u % splits; parted = partial != nullptr; }
    };

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 256); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tmA) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tmB) : "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(tmem_slot)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();          // the peer's barriers exist before anything is signalled across the pair
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            int it = 0;
            bool first = true, ok = true;
            for (int t = pair; t < total && ok; t += num_pairs) {
                int tile, split;
                bool parted;
                item_of(t, tile, split, parted);
                const int tm = tile % tiles_m, tn = tile / tiles_m;
                const int arow = tm * 256 + (int)rank * 128, brow = tn * BN + (int)rank * 128;
                const int kb0 = parted ? split * kb_per_split : 0, kb1 = parted ? min(num_kb, kb0 + kb_per_split) : num_kb;
                int kb = kb0;
                if (first) {
                    const int pre = kb1 - kb0 < STAGES ? kb1 - kb0 : STAGES;
                    for (int i = 0; i < pre; ++i) {
                        if (leader) mbar_expect_tx(&full[i], 2 * STAGE_BYTES);
                        tma_load_2d_pair(smem + i * STAGE_BYTES + A_BYTES, &tmB, &full[i], (kb0 + i) * BK, brow);
                    }
                    pdl_wait();
                    for (int i = 0; i < pre; ++i) tma_load_2d_pair(smem + i * STAGE_BYTES, &tmA, &full[i], (kb0 + i) * BK, arow);
                    kb = kb0 + pre;
                    it = pre;
                    first = false;
                }
                for (; kb < kb1; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (uint32_t)(it / STAGES) & 1u;
                    if (!mbar_wait(&empty[s], ph ^ 1u, abort_flag, status, 1)) { ok = false; break; }
                    if (leader) mbar_expect_tx(&full[s], 2 * STAGE_BYTES);
                    uint8_t* sa = smem + s * STAGE_BYTES;
                    tma_load_2d_pair(sa, &tmA, &full[s], kb * BK, arow);
                    tma_load_2d_pair(sa + A_BYTES, &tmB, &full[s], kb * BK, brow);
                }
            }
            if (first) pdl_wait();
        }
    } else if (warp == 1) {
        if (lane == 0 && leader) {
            const uint32_t idesc = make_idesc(256, BN);
            int it = 0, i = 0;
            bool ok = true;
            for (int t = pair; t < total && ok; t += num_pairs, ++i) {
                const int buf = i & 1;
                const uint32_t aph = (uint32_t)(i >> 1) & 1u;
                ok = mbar_wait(&acc_empty[buf], aph ^ 1u, abort_flag, status, 4);
                if (!ok) break;
                tc_fence_after();
                const uint32_t tacc = tmem_base + (uint32_t)(buf * BN);
                int tile, split;
                bool parted;
                item_of(t, tile, split, parted);
                const int kb0 = parted ? split * kb_per_split : 0, kb1 = parted ? min(num_kb, kb0 + kb_per_split) : num_kb;
                for (int kb = kb0; kb < kb1; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (uint32_t)(it / STAGES) & 1u;
                    ok = mbar_wait(&full[s], ph, abort_flag, status, 2);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t sa = smem_u32(smem + s * STAGE_BYTES);
                    const uint64_t adesc = make_smem_desc(sa);
                    const uint64_t bdesc = make_smem_desc(sa + A_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)
                        umma_pair(tacc, adesc + 2 * k, bdesc + 2 * k, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
                    umma_commit_pair(&empty[s]);
                }
                if (ok) umma_commit_pair(&acc_full[buf]);
            }
        }
    } else {
        const int q = warp & 3;
        const int row = q * 32 + lane;
        pdl_wait();
        int i = 0;
        for (int t = pair; t < total; t += num_pairs, ++i) {
            int tile, split;
            bool parted;
            item_of(t, tile, split, parted);
            const int tm = tile % tiles_m, tn = tile / tiles_m;
            const int buf = i & 1;
            const uint32_t aph = (uint32_t)(i >> 1) & 1u;
            const int gi = tm * 256 + (int)rank * 128 + row;
            const float sc = (gi < M && !parted) ? norm_factor(nio, gi) : 1.0f;   // while the tile is still being multiplied
            if (!mbar_wait(&acc_full[buf], aph, abort_flag, status, 3)) break;
            tc_fence_after();
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * BN);
            if (parted) {
                // the raw sums of this K range: row gi of split's [M][NS] float32 tile
                float* prow = partial + ((size_t)split * M + gi) * NS + (tn - tn_split) * BN;
#pragma unroll 1
                for (int c0 = 0; c0 < BN; c0 += 16) {
                    if (tn * BN + c0 >= N) break;
                    uint32_t r[16];
                    tmem_ld16(taddr + (uint32_t)c0, r);
                    tmem_ld_wait();
                    if (gi >= M) continue;
                    if (tn * BN + c0 + 16 <= N && ((((uintptr_t)(prow + c0)) & 15) == 0)) {
#pragma unroll
                        for (int j = 0; j < 4; ++j)
                            reinterpret_cast<float4*>(prow + c0)[j] = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                                                                 __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (tn * BN + c0 + j < N) prow[c0 + j] = __uint_as_float(r[j]);
                    }
                }
            } else if (out_mode == OUT_QKV)
                epilogue_row_qkv(taddr, gi, tn, M, qio, sc);
            else
                epilogue_row_256(taddr, gi, tn, M, N, out, out_mode, ldo, nio, sc);
            tc_fence_before();
            mbar_arrive_cluster(&acc_empty[buf], 0);     // 256 arrivals in the leader free the accumulator pair
        }
    }

    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000LL) { }
        __syncthreads();
    }
    cluster_sync_all();          // neither CTA leaves while the other may still signal its barriers
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
    }
}

// out (mode) = sum over splits of partial[s], scaled by the folded norm's factor: a warp per (token, block of 128
// columns), the epilogue of the decode form.  The partial tiles cover the columns from `col0` on (the tile columns
// that were split), NS of them per row.
__global__ void __launch_bounds__(256) gemm_splitk_finish_kernel(const float* partial, int splits, void* __restrict__ out,
                                                                 int out_mode, long long ldo, int M, int N, int col0, int NS,
                                                                 const NormIO nio, const QkvIO qio) {
    pdl_launch();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int gj = blockIdx.y * 8 + (threadIdx.x >> 5);          // token
    const int tile_a = col0 / 128 + blockIdx.x;                  // block of 128 columns
    if (gj >= M) return;
    const int c0 = tile_a * 128 + 4 * lane;
    QkvTok qt;
    if (out_mode == OUT_QKV) qt = qkv_token_data(qio, gj, tile_a, lane);       // a block of 128 columns is one head
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    if (c0 + 4 <= N && (NS & 3) == 0) {
        for (int s = 0; s < splits; ++s) {
            const float4 v = *reinterpret_cast<const float4*>(partial + ((size_t)s * M + gj) * NS + (c0 - col0));
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
    } else {
        float f[4] = {0.f, 0.f, 0.f, 0.f};
        for (int s = 0; s < splits; ++s)
            for (int t = 0; t < 4; ++t)
                if (c0 + t < N) f[t] += partial[((size_t)s * M + gj) * NS + (c0 - col0) + t];
        acc = make_float4(f[0], f[1], f[2], f[3]);
    }
    if (nio.in_ssq != nullptr) {
        const float sc = norm_factor_warp(nio, gj, lane);
        acc.x *= sc; acc.y *= sc; acc.z *= sc; acc.w *= sc;
    }
    if (out_mode == OUT_QKV) {
        qkv_token_finish(acc, gj, tile_a, lane, qio, qt);
        return;
    }
    finish_token_block(acc, gj, tile_a, lane, out, out_mode, ldo, N, nio);
}

// Work items of the CTA-pair form for a product whose tiles do not fill the 74 pairs well.  `splits` > 1: the K range
// of a tile is split that many ways; `whole`: the first tiles (in tile order; a multiple of the tile rows, so
// whole tile columns) that are not split.  Two shapes of plan: every tile split (few tiles: prompts of a few
// hundred tokens), or the full waves whole and only the tiles of a last wave that is less than half full split.  Every split
// keeps eight 64-wide slabs, and the float32 partial tiles (written and read once, then a second kernel) must cost
// less than the idle pairs.  {1, tiles}: no split.
struct PairPlan {
    int splits;
    int whole;
    long long scratch_elems(int M, int N) const {
        if (splits <= 1) return 0;
        const int tiles_m = (M + 255) / 256;
        return (long long)splits * M * (N - (whole / tiles_m) * 256);
    }
};
PairPlan pair_plan(int M, int N, int K, bool uneven_ok) {
    const int tiles_m = (M + 255) / 256, tiles = tiles_m * ((N + 255) / 256);
    const int num_kb = (K + BK - 1) / BK;
    const int pairs = 74;
    // time of the product in units of seconds: a 256 x 256 x K tile takes about 2 * 256 * 256 * K / (1.3e15 / 74) s;
    // 6e12 bytes/s for the partial tiles
    const double tile_s = 2.0 * 256 * 256 * K / (1.3e15 / pairs);
    double best_cost = 1e30;
    PairPlan best = {1, tiles};
    for (int s = 1; s <= 8; ++s) {
        if (s > 1 && num_kb / s < 8) break;
        const int items = tiles * s;
        const int waves = (items + pairs - 1) / pairs;
        const double cost = waves * tile_s / s + (s > 1 ? 2.0 * s * M * (double)N * 4 / 6e12 : 0.0);
        if (cost < best_cost * 0.97) { best_cost = cost; best = PairPlan{s, s > 1 ? 0 : tiles}; }
    }
    // The second shape, for products in the compute-bound range (more than 768 tokens; measured: the gate-up product
    // of 256 tokens, which streams its weights at the memory's rate, gains nothing from it).  The pairs walk the
    // items round-robin, whole tiles first, so the estimate is the longest pair's sum of its items.
    if (uneven_ok && tiles > pairs && tiles_m >= 4) {
        const int base = ((tiles / pairs) * pairs / tiles_m) * tiles_m;       // the full waves, in whole tile columns
        for (int whole = base; whole > 0 && whole > base - 2 * tiles_m; whole -= tiles_m) {
            const int rest = tiles - whole;
            if (rest > pairs / 2) continue;       // (measured: with a last wave more than half full the split gains nothing)
            for (int s = 2; s <= 4 && rest > 0; ++s) {
                if (num_kb / s < 8) break;
                const int total = whole + rest * s;
                double longest = 0.0;
                for (int p = 0; p < pairs; ++p) {
                    double sum = 0.0;
                    for (int t = p; t < total; t += pairs) sum += t < whole ? tile_s : tile_s / s + 3e-6;
                    if (sum > longest) longest = sum;
                }
                const double cols = (double)(rest / tiles_m) * 256;
                const double cost = longest + 2.0 * s * M * cols * 4 / 6e12 + 4e-6;
                if (cost < best_cost * 0.97) { best_cost = cost; best = PairPlan{s, whole}; }
            }
        }
    }
    return best;
}

int launch_pair(const CUtensorMap& ta, const CUtensorMap& tb, void* out, int out_mode, long long ldo, int M, int N,
                int K, int* status, const NormIO& nio, const QkvIO& qio, PairPlan plan, float* partial, cudaStream_t stream) {
    constexpr int STAGES = 6;
    constexpr int smem = STAGES * (A_BYTES + 128 * BK * 2) + 1024 + 256;
    static int sms = 0;
    auto kern = gemm_tc_pair_kernel<STAGES>;
    if (sms == 0) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return (int)e;
        int dev = 0, n = 0;
        if ((e = cudaGetDevice(&dev)) != cudaSuccess) return (int)e;
        if ((e = cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return (int)e;
        sms = n > 0 ? n : 148;
    }
    const int tiles_m = (M + 255) / 256, tiles = tiles_m * ((N + 255) / 256);
    const int num_kb = (K + BK - 1) / BK;
    const int per = (num_kb + plan.splits - 1) / plan.splits;
    const int used = (num_kb + per - 1) / per;           // no empty split
    int whole = plan.whole;
    if (used == 1) { partial = nullptr; whole = tiles; }
    const int total = whole + (tiles - whole) * used;
    int pairs = sms / 2;
    if (pairs > total) pairs = total;
    int rc = gg_launch2(kern, dim3(2 * pairs), dim3(NUM_THREADS), smem, stream, ta, tb, out, out_mode, ldo, M, N, K, status, nio,
                        used, whole, per, partial, qio);
    if (rc != 0 || used == 1) return rc;
    const int col0 = (whole / tiles_m) * 256, NS = N - col0;
    return gg_launch(gemm_splitk_finish_kernel, dim3((NS + 127) / 128, (M + 7) / 8), dim3(256), 0, stream, 1,
                     (const float*)partial, used, out, out_mode, ldo, M, N, col0, NS, nio, qio);
}

template <int BN, int STAGES, bool SWAP, int MINB>
int launch(const CUtensorMap& ta, const CUtensorMap& tb, void* out, int out_mode, long long ldo, int M, int N, int K,
           int splits, int kb_per_split, float* partial, bool cluster, int* status, const NormIO& nio,
           const QkvIO& qio, cudaStream_t stream) {
    constexpr int smem = STAGES * (A_BYTES + BN * BK * 2) + 1024 + 256 + recv_bytes<BN, SWAP>() + (SWAP && BN > 16 ? 512 : 0);
    static_assert(STAGES * (A_BYTES + BN * BK * 2) >= BN * BM * 4, "the stages must hold a float32 tile");
    static_assert(!SWAP || BN != 32 || STAGES * (A_BYTES + BN * BK * 2) >= (2 * BN + MAX_CLUSTER - 1) * BM * 4,
                  "at 32 tokens the stages must also hold what the other ranks push");
    static bool configured = false;
    auto kern = gemm_tc_kernel<BN, STAGES, SWAP, MINB>;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    const int RA = SWAP ? N : M, RB = SWAP ? M : N;
    dim3 grid((RA + BM - 1) / BM, (RB + BN - 1) / BN, splits);
    float* part = (splits > 1 && !cluster) ? partial : nullptr;
    const int cl = (splits > 1 && cluster) ? 1 : 0;
    if (!SWAP && (cl || out_mode == OUT_SWIGLU || out_mode == OUT_QKV)) return GG_ERR_ARG;      // forms the normal orientation does not have
    return gg_launch(kern, grid, dim3(NUM_THREADS), smem, stream, cl ? splits : 1, ta, tb, out, out_mode, ldo, M, N, K,
                     kb_per_split, part, cl, status, nio, qio);
}

}  // namespace

// Number of K splits the launcher uses for a product of this shape (0: the shape is not taken).
// use_cluster != 0: the splits of a tile form a thread-block cluster (at most 8) and no scratch is
// needed.  use_cluster == 0: partial sums go through a scratch buffer of splits * M * N floats.
GG_API gg_gemm_tc_splits(int M, int N, int K, int use_cluster) {
    if (M <= 0 || N <= 0 || K <= 0 || (K % 8) != 0) return 0;
    if (M > 128) return 1;
    const int num_kb = (K + BK - 1) / BK;
    const int tiles = (N + BM - 1) / BM;
    const int per_sm = 3;                        // CTAs that share an SM in the decode forms
    int splits = (148 * per_sm + tiles / 2) / tiles;
    if (splits > num_kb / 2) splits = num_kb / 2;  // at least two 64-wide slabs per CTA
    const int most = use_cluster ? MAX_CLUSTER : 16;
    if (splits > most) splits = most;
    if (splits < 1) splits = 1;
    // no empty split: the last one must own at least one slab
    int per = (num_kb + splits - 1) / splits;
    splits = (num_kb + per - 1) / per;
    return splits;
}

// out[M, N] (mode) = x[M, K] (bf16, row stride ldx) * w[N, K]^T (bf16, contiguous).
// out_mode: 0 bf16 store, 1 float32 store, 2 float32 add (residual), 3 fused SwiGLU (see below).
// use_cluster != 0: K splits are reduced inside thread-block clusters; scratch is not touched.
// use_cluster == 0: scratch must hold gg_gemm_tc_splits(M, N, K, 0) * M * N floats when that count is > 1.
// status: one int on the device, zero-initialised by the caller; a non-zero value after the kernel
// means a bounded wait ran out (1 producer, 2 issuer, 3 epilogue).
static int gemm_tc_impl(const void* x, const void* w, void* out, int out_mode, int M, int N, int K, long long ldx,
                        long long ldo, float* scratch, long long scratch_elems, int use_cluster, int* status,
                        const NormIO& nio, const QkvIO& qio, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || (K % 8) != 0 || (ldx % 8) != 0 || ldx < K || out_mode < 0 || out_mode > 4) return GG_ERR_ARG;
    if (out_mode == OUT_QKV) {
        // one 128-wide head per weight tile (decode form) or two per tile (CTA-pair form); `out` is not used
        if (qio.nq <= 0 || qio.nkv <= 0 || N != (qio.nq + 2 * qio.nkv) * 128 || qio.q_out == nullptr ||
            qio.cosv == nullptr || qio.sinv == nullptr || qio.positions == nullptr || qio.seq_of_token == nullptr ||
            (qio.k_pool != nullptr && (qio.v_pool == nullptr || qio.page_table == nullptr || qio.page_size <= 0)))
            return GG_ERR_ARG;
        const uintptr_t al = (uintptr_t)qio.q_out | (uintptr_t)qio.k_pool | (uintptr_t)qio.v_pool | (uintptr_t)qio.cosv |
                             (uintptr_t)qio.sinv | (uintptr_t)qio.qw | (uintptr_t)qio.kw;
        if (al & 15) return GG_ERR_ARG;
        ldo = N;
        use_cluster = 1;
    }
    // out_mode 3: w holds blocks of 64 gate rows and 64 up rows in turn; out[M, N / 2] (bf16) = silu(gate) * up
    if (out_mode == OUT_SWIGLU ? ((N % 128) != 0 || ldo < N / 2 || (M > 128 && N < 256)) : ldo < N) return GG_ERR_ARG;
    if ((((uintptr_t)x) & 15) || (((uintptr_t)w) & 15) || status == nullptr) return GG_ERR_ARG;
    const int num_kb = (K + BK - 1) / BK;
    const bool swap = M <= 128;
    if (out_mode == OUT_SWIGLU) use_cluster = 1;      // the fused activation needs the staged reduction
    const bool cluster = use_cluster != 0;
    int splits = gg_gemm_tc_splits(M, N, K, use_cluster);
    if (splits > 1 && !cluster && (scratch == nullptr || scratch_elems < (long long)splits * M * N)) return GG_ERR_ARG;
    const int per = (num_kb + splits - 1) / splits;
    CUtensorMap ta, tb;
    int rc;
    if (swap) {
        const int bn = M <= 16 ? 16 : (M <= 32 ? 32 : (M <= 64 ? 64 : 128));
        if ((rc = make_map(&ta, w, N, K, K, BM)) != 0) return rc;
        if ((rc = make_map(&tb, x, M, K, ldx, bn)) != 0) return rc;
        // A grid that fits two CTAs per SM (296 places) gets the deeper ring; a larger one needs three per SM
        // to run as one wave.  GOGGUF_B200_GEMM_DEEP=0 always takes the three-per-SM forms.
        static int deep_ok = -1;
        if (deep_ok < 0) { const char* e = getenv("GOGGUF_B200_GEMM_DEEP"); deep_ok = (e != nullptr && e[0] == '0') ? 0 : 1; }
        const long long ctas = (long long)((N + BM - 1) / BM) * ((M + bn - 1) / bn) * splits;
        const bool deep = deep_ok && ctas <= 296 && bn <= 32;    // measured in whole steps: a gain up to 32 tokens only
#define GG_DECODE(BN_, ST_, MINB_) launch<BN_, ST_, true, MINB_>(ta, tb, out, out_mode, ldo, M, N, K, splits, per, scratch, \
                                                                 cluster, status, nio, qio, stream)
        if (bn == 16) rc = deep ? GG_DECODE(16, 5, 2) : GG_DECODE(16, 3, 3);     // stages + the receive area fill the SM
        else if (bn == 32) rc = deep ? GG_DECODE(32, 5, 2) : GG_DECODE(32, 3, 3);
        else if (bn == 64) rc = deep ? GG_DECODE(64, 4, 2) : GG_DECODE(64, 3, 3);
        else rc = deep ? GG_DECODE(128, 3, 2) : GG_DECODE(128, 2, 3);
#undef GG_DECODE
    } else {
        const int bn = N > 128 ? 256 : 128;
        if ((rc = make_map(&ta, x, M, K, ldx, BM)) != 0) return rc;
        if ((rc = make_map(&tb, w, N, K, K, bn)) != 0) return rc;
        static int use_pair = -1;
        if (use_pair < 0) { const char* e = getenv("GOGGUF_B200_GEMM_PAIR"); use_pair = (e != nullptr && e[0] == '0') ? 0 : 1; }
        if (bn == 256 && use_pair) {
            // CTA pairs: A tiles of 128 rows per CTA as before, B staged in halves of 128 rows per CTA
            if ((rc = make_map(&tb, w, N, K, K, 128)) != 0) return rc;
            // (a split q/k/v product leaves the per-head epilogue to the kernel that adds the partial tiles)
            PairPlan plan = pair_plan(M, N, K, true);
            if (plan.splits > 1 && (scratch == nullptr || scratch_elems < plan.scratch_elems(M, N)))
                plan = PairPlan{1, 0};                                                   // no room for partial tiles
            rc = launch_pair(ta, tb, out, out_mode, ldo, M, N, K, status, nio, qio, plan, scratch, stream);
        } else if (out_mode == OUT_QKV) rc = GG_ERR_ARG;       // only the CTA-pair form has the q/k/v epilogue
        else if (bn == 256) rc = launch_persistent(ta, tb, out, out_mode, ldo, M, N, K, status, nio, stream);
        else rc = launch<128, 6, false, 1>(ta, tb, out, out_mode, ldo, M, N, K, 1, per, scratch, false, status, nio, qio, stream);
    }
    if (rc != 0) return rc;
    if (splits > 1 && !cluster) {
        const long long total = (long long)M * N;
        return gg_launch(splitk_reduce_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, 1,
                         (const float*)scratch, out, out_mode, ldo, M, N, splits);
    }
    return 0;
}

GG_API gg_gemm_tc(const void* x, const void* w, void* out, int out_mode, int M, int N, int K, long long ldx,
                  long long ldo, float* scratch, long long scratch_elems, int use_cluster, int* status,
                  cudaStream_t stream) {
    if (out_mode == OUT_QKV) return GG_ERR_ARG;
    const NormIO none = {nullptr, 0, 0.f, 0.f, nullptr, nullptr};
    const QkvIO noq = {};
    return gemm_tc_impl(x, w, out, out_mode, M, N, K, ldx, ldo, scratch, scratch_elems, use_cluster, status, none, noq, stream);
}

// The same product with an RMSNorm folded in on either side (K splits always inside clusters).
//   in_ssq != null: x is the bfloat16 copy of the raw residual rows, w already carries the norm's weight,
//     in_ssq[M, in_parts] holds partial sums of squares of those rows (in_parts = ceil(K / 128)); every
//     accumulator row is multiplied by 1 / sqrt(sum / K + eps) before the output mode is applied.
//   scratch: optional room for the float32 partial tiles of a K split at more than 128 tokens
//     (gg_gemm_tc_pair_scratch_elems).
//   out_ssq != null (out_mode 2 only): after out += product the kernel also writes out_xhat[M, N]
//     (bfloat16 copy of the updated rows, row stride N) and out_ssq[M, ceil(N / 128)], their partial sums
//     of squares over blocks of 128 columns: the inputs of the next folded product.
GG_API gg_gemm_tc_norm(const void* x, const void* w, void* out, int out_mode, int M, int N, int K, long long ldx,
                       long long ldo, const float* in_ssq, int in_parts, float eps, float* out_ssq, void* out_xhat,
                       float* scratch, long long scratch_elems, int* status, cudaStream_t stream) {
    if (in_ssq != nullptr && (in_parts != (K + 127) / 128 || !(eps > 0.f))) return GG_ERR_ARG;
    if (out_ssq != nullptr && (out_mode != OUT_F32_ACC || out_xhat == nullptr)) return GG_ERR_ARG;
    if (out_mode == OUT_QKV) return GG_ERR_ARG;
    const NormIO nio = {in_ssq, in_parts, 1.0f / (float)K, eps, out_ssq, (bf16*)out_xhat};
    const QkvIO noq = {};
    return gemm_tc_impl(x, w, out, out_mode, M, N, K, ldx, ldo, scratch, scratch_elems, 1, status, nio, noq, stream);
}

// Floats of scratch with which a product of more than 128 tokens splits K over CTA pairs (0: it would not split).
// Without that much scratch the product runs unsplit.
GG_API gg_gemm_tc_pair_scratch_elems(int M, int N, int K, long long* elems) {
    if (elems == nullptr) return GG_ERR_ARG;
    *elems = 0;
    if (M <= 128 || N <= 128 || K <= 0) return 0;
    *elems = pair_plan(M, N, K, true).scratch_elems(M, N);
    return 0;
}

// The q/k/v projection of a step (head size 128; more than 128 tokens in the CTA-pair form) with the per-head q/k RMSNorm,
// the rotation and the cache write in its epilogue: x[M, K] * w[(nq + 2 nkv) * 128, K]^T, rows of w being
// all q heads, then all k heads, then all v heads.  See QkvIO for the outputs; in_ssq / in_parts / in_eps
// as in gg_gemm_tc_norm (null: x is already normalised).  qw / kw null: no q/k norm.
GG_API gg_gemm_tc_qkv_rope(const void* x, const void* w, int M, int K, long long ldx, const float* in_ssq, int in_parts,
                           float in_eps, void* q_out, const float* qw, const float* kw, float eps, const float* cosv,
                           const float* sinv, const int* positions, const int* seq_of_token, const int* page_table,
                           int max_pages, int page_size, int n_pages, void* k_pool, void* v_pool, int nq, int nkv,
                           float* scratch, long long scratch_elems, int* status, cudaStream_t stream) {
    if (in_ssq != nullptr && (in_parts != (K + 127) / 128 || !(in_eps > 0.f))) return GG_ERR_ARG;
    const NormIO nio = {in_ssq, in_parts, K > 0 ? 1.0f / (float)K : 0.f, in_eps, nullptr, nullptr};
    const QkvIO qio = {(bf16*)q_out, qw, kw, eps, cosv, sinv, positions, seq_of_token, page_table, max_pages, page_size,
                       (bf16*)k_pool, (bf16*)v_pool, nq, nkv, n_pages, status};
    const int N = (nq + 2 * nkv) * 128;
    return gemm_tc_impl(x, w, q_out, OUT_QKV, M, N, K, ldx, N, scratch, scratch_elems, 1, status, nio, qio, stream);
}
