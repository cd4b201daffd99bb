// On-device sampling from float32 logits: greedy and temperature.
//
// greedy: the first index of the maximum (strict '>', pkg/sampler/greedy.go:4-17).
// temperature: x = float32(float64(logit) / temp) (pkg/sampler/probs.go:40-49); softmax with
// the maximum subtracted in float32 and exp and sum in float64 (probs.go:20-38); the draw walks
// the ids in order, r = u * sum(p), and returns the first id at which the running sum reaches r
// (pkg/sampler/chain.go:135-166), the last id if rounding leaves r above the total.
// The uniform number u of each row is given by the caller (a counter-based generator keyed by
// request and step), so a sequence's draws do not depend on its neighbours in the batch.
#include "common.cuh"

#define SAMP_THREADS 1024

struct MaxIdx { float v; int i; };

__device__ __forceinline__ MaxIdx better(MaxIdx a, MaxIdx b) {
    // larger value wins; equal values: smaller index wins (first maximum)
    if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
    return a;
}

__device__ __forceinline__ MaxIdx block_argmax(MaxIdx x, MaxIdx* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        MaxIdx y;
        y.v = __shfl_xor_sync(0xffffffffu, x.v, o);
        y.i = __shfl_xor_sync(0xffffffffu, x.i, o);
        x = better(x, y);
    }
    __syncthreads();
    if (lane == 0) red[warp] = x;
    __syncthreads();
    if (warp == 0) {
        MaxIdx t = lane < nw ? red[lane] : MaxIdx{-INFINITY, 0x7fffffff};
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            MaxIdx y;
            y.v = __shfl_xor_sync(0xffffffffu, t.v, o);
            y.i = __shfl_xor_sync(0xffffffffu, t.i, o);
            t = better(t, y);
        }
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}

__device__ __forceinline__ double block_sum_f64(double v, double* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    if (warp == 0) {
        double t = lane < nw ? red[lane] : 0.0;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}

__global__ void __launch_bounds__(SAMP_THREADS) argmax_kernel(const float* logits, long long ld,
                                                               int* __restrict__ out, int V) {
    pdl_launch();
    pdl_wait();
    __shared__ MaxIdx red[33];
    const float* x = logits + (size_t)blockIdx.x * ld;
    MaxIdx best{-INFINITY, 0x7fffffff};
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float v = x[i];
        if (v > best.v || best.i == 0x7fffffff) best = MaxIdx{v, i};
    }
    best = block_argmax(best, red);
    if (threadIdx.x == 0) out[blockIdx.x] = best.i == 0x7fffffff ? 0 : best.i;
}

// Two-stage form for a few long rows: `chunks` blocks per row each find the best of their slice, a second
// launch picks among them (ties still go to the smallest index).
__global__ void __launch_bounds__(SAMP_THREADS) argmax_partial_kernel(const float* logits, long long ld,
                                                                       MaxIdx* __restrict__ part, int V, int chunks) {
    pdl_launch();
    pdl_wait();
    __shared__ MaxIdx red[33];
    const int r = blockIdx.x, c = blockIdx.y;
    const float* x = logits + (size_t)r * ld;
    const int per = ((V + chunks - 1) / chunks + 3) & ~3;
    const int lo = c * per, hi = min(V, lo + per);
    MaxIdx best{-INFINITY, 0x7fffffff};
    for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
        const float v = x[i];
        if (v > best.v || best.i == 0x7fffffff) best = MaxIdx{v, i};
    }
    best = block_argmax(best, red);
    if (threadIdx.x == 0) part[(size_t)r * chunks + c] = best;
}

__global__ void argmax_final_kernel(const MaxIdx* part, int* __restrict__ out, int chunks) {
    pdl_launch();
    pdl_wait();
    const int r = blockIdx.x;
    MaxIdx best{-INFINITY, 0x7fffffff};
    for (int c = threadIdx.x; c < chunks; c += 32) best = better(best, part[(size_t)r * chunks + c]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        MaxIdx y;
        y.v = __shfl_xor_sync(0xffffffffu, best.v, o);
        y.i = __shfl_xor_sync(0xffffffffu, best.i, o);
        best = better(best, y);
    }
    if (threadIdx.x == 0) out[r] = best.i == 0x7fffffff ? 0 : best.i;
}

// scratch: at least R * 64 pairs of (float, int) = R * 128 four-byte words, or null for the one-block form.
GG_API gg_argmax(const float* logits, long long ld, int* out, int R, int V, void* scratch, long long scratch_words,
                 cudaStream_t stream) {
    if (R <= 0) return 0;
    if (V <= 0 || ld < V) return GG_ERR_ARG;
    int chunks = 1;
    if (scratch != nullptr && V >= 16384) {
        chunks = 592 / R;                       // about four blocks per SM in all
        if (chunks > 64) chunks = 64;
        if (chunks > V / 4096) chunks = V / 4096;
        if ((long long)R * chunks * 2 > scratch_words) chunks = 1;
    }
    if (chunks <= 1) {
        gg_launch(argmax_kernel, dim3(R), dim3(SAMP_THREADS), 0, stream, 1, logits, ld, out, V);
        return gg_last_error();
    }
    dim3 grid(R, chunks);
    gg_launch(argmax_partial_kernel, dim3(grid), dim3(SAMP_THREADS), 0, stream, 1, logits, ld, (MaxIdx*)scratch, V, chunks);
    gg_launch(argmax_final_kernel, dim3(R), dim3(32), 0, stream, 1, (const MaxIdx*)scratch, out, chunks);
    return gg_last_error();
}

// One block per row.  temps[r] <= 0 means greedy for that row.
__global__ void __launch_bounds__(SAMP_THREADS) sample_kernel(const float* logits, long long ld,
                                                               const float* __restrict__ temps,
                                                               const double* __restrict__ uniforms,
                                                               int* __restrict__ out, int V) {
    pdl_launch();
    pdl_wait();
    __shared__ MaxIdx red[33];
    __shared__ double dred[33];
    __shared__ double pre[SAMP_THREADS];
    __shared__ int found;
    const int r = blockIdx.x;
    const float* x = logits + (size_t)r * ld;
    const float temp = temps[r];
    const bool scaled = temp > 0.f && temp != 1.f;
    const double inv_t = scaled ? 1.0 / (double)temp : 1.0;

    MaxIdx best{-INFINITY, 0x7fffffff};
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float v = scaled ? (float)((double)x[i] * inv_t) : x[i];
        if (v > best.v || best.i == 0x7fffffff) best = MaxIdx{v, i};
    }
    best = block_argmax(best, red);
    if (temp <= 0.f) {
        if (threadIdx.x == 0) out[r] = best.i == 0x7fffffff ? 0 : best.i;
        return;
    }
    const float mx = best.v;
    // contiguous chunk per thread so that the running sum follows the id order
    const int chunk = (V + blockDim.x - 1) / blockDim.x;
    const int lo = threadIdx.x * chunk;
    const int hi = min(V, lo + chunk);
    double local = 0.0;
    for (int i = lo; i < hi; ++i) {
        const float v = scaled ? (float)((double)x[i] * inv_t) : x[i];
        local += exp((double)(v - mx));
    }
    const double total = block_sum_f64(local, dred);
    const double inv = 1.0 / total;
    // exclusive prefix over threads (sequential by one thread: 1024 additions, fixed order)
    pre[threadIdx.x] = local * inv;
    if (threadIdx.x == 0) found = 0x7fffffff;
    __syncthreads();
    if (threadIdx.x == 0) {
        double run = 0.0;
        for (int t = 0; t < (int)blockDim.x; ++t) { const double c = pre[t]; pre[t] = run; run += c; }
        dred[0] = run;  // sum of the normalised probabilities
    }
    __syncthreads();
    const double target = uniforms[r] * dred[0];
    double run = pre[threadIdx.x];
    if (lo < hi && run < target + 1e-300) {
        // the crossing can only lie in this chunk if the running sum before it is below the target
        for (int i = lo; i < hi; ++i) {
            const float v = scaled ? (float)((double)x[i] * inv_t) : x[i];
            run += exp((double)(v - mx)) * inv;
            if (target - run <= 0.0) { atomicMin(&found, i); break; }
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) out[r] = found == 0x7fffffff ? V - 1 : found;
}

GG_API gg_sample(const float* logits, long long ld, const float* temps, const double* uniforms, int* out,
                 int R, int V, cudaStream_t stream) {
    if (R <= 0) return 0;
    if (V <= 0 || ld < V) return GG_ERR_ARG;
    gg_launch(sample_kernel, dim3(R), dim3(SAMP_THREADS), 0, stream, 1, logits, ld, temps, uniforms, out, V);
    return gg_last_error();
}
