// Plain matrix product on the CUDA cores: out[M,N] (+)= x[M,K] * W[N,K]^T, float32 accumulate.
//
// This is the true 32-bit path of every projection (no tensor cores, no reduced
// precision mode) and the plain twin the tensor-core kernels are checked against.
// It also serves mixed operands (bfloat16 activations with a matrix that is stored
// in 32-bit and stays so).  Each output element is accumulated over k in a fixed
// order that does not depend on M, so a token's result does not depend on the batch.
// The reference's counterpart is the one-thread-per-row matmul_vec PTX kernel
// (pkg/gpu/cuda/ptx.go:67-129) and ops.MatMulVecInto (pkg/ops/ops.go:30-53).
#include "common.cuh"

#define BM 64
#define BN 64
#define BK 16

template <typename TX, typename TW, typename TO, bool ACC>
__global__ void __launch_bounds__(256) gemm_plain_kernel(const TX* x, const TW* __restrict__ w,
                                                         TO* __restrict__ out, int M, int N, int K,
                                                         long long ldx, long long ldo) {
    pdl_launch();
    pdl_wait();
    __shared__ float xs[BK][BM + 1];
    __shared__ float ws[BK][BN + 1];
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int tid = threadIdx.x;
    const int tm = (tid / 16) * 4, tn = (tid % 16) * 4;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += BK) {
        // 64 rows x 16 k = 1024 elements per operand, 4 per thread
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int idx = tid + e * 256;
            const int r = idx / BK, kk = idx % BK;
            const int gk = k0 + kk;
            float xv = 0.f, wv = 0.f;
            if (gk < K) {
                if (m0 + r < M) xv = to_f<TX>(x[(size_t)(m0 + r) * ldx + gk]);
                if (n0 + r < N) wv = to_f<TW>(w[(size_t)(n0 + r) * K + gk]);
            }
            xs[kk][r] = xv;
            ws[kk][r] = wv;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = xs[kk][tm + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = ws[kk][tn + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
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
            TO* o = out + (size_t)m * ldo + n;
            if (ACC) *o = from_f<TO>(to_f<TO>(*o) + acc[i][j]);
            else *o = from_f<TO>(acc[i][j]);
        }
    }
}

template <typename TX, typename TW>
static int launch(const void* x, const void* w, void* out, int out_dtype, int accumulate,
                  int M, int N, int K, long long ldx, long long ldo, cudaStream_t stream) {
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    if (out_dtype == GG_F32) {
        if (accumulate) gg_launch(gemm_plain_kernel<TX, TW, float, true>, dim3(grid), dim3(256), 0, stream, 1, (const TX*)x, (const TW*)w, (float*)out, M, N, K, ldx, ldo);
        else gg_launch(gemm_plain_kernel<TX, TW, float, false>, dim3(grid), dim3(256), 0, stream, 1, (const TX*)x, (const TW*)w, (float*)out, M, N, K, ldx, ldo);
    } else if (out_dtype == GG_BF16) {
        if (accumulate) return GG_ERR_DTYPE;  // sums are kept in float32
        gg_launch(gemm_plain_kernel<TX, TW, bf16, false>, dim3(grid), dim3(256), 0, stream, 1, (const TX*)x, (const TW*)w, (bf16*)out, M, N, K, ldx, ldo);
    } else {
        return GG_ERR_DTYPE;
    }
    return gg_last_error();
}

// x[M, K] with row stride ldx (elements), w[N, K] contiguous, out[M, N] with row stride ldo.
// accumulate != 0: out += product (float32 out only; this is the residual add).
GG_API gg_gemm_plain(const void* x, int x_dtype, const void* w, int w_dtype, void* out, int out_dtype,
                     int accumulate, int M, int N, int K, long long ldx, long long ldo, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || ldx < K || ldo < N) return GG_ERR_ARG;
    if ((M + BM - 1) / BM > 65535) return GG_ERR_ARG;
    if (x_dtype == GG_F32 && w_dtype == GG_F32) return launch<float, float>(x, w, out, out_dtype, accumulate, M, N, K, ldx, ldo, stream);
    if (x_dtype == GG_BF16 && w_dtype == GG_BF16) return launch<bf16, bf16>(x, w, out, out_dtype, accumulate, M, N, K, ldx, ldo, stream);
    if (x_dtype == GG_BF16 && w_dtype == GG_F32) return launch<bf16, float>(x, w, out, out_dtype, accumulate, M, N, K, ldx, ldo, stream);
    if (x_dtype == GG_F32 && w_dtype == GG_BF16) return launch<float, bf16>(x, w, out, out_dtype, accumulate, M, N, K, ldx, ldo, stream);
    return GG_ERR_DTYPE;
}
