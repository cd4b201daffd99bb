// On-device sampling from float32 logits: greedy, temperature, and the whole chain of masks when a
// top-k is set (temperature, top-k, min-p, softmax, top-p, draw: pkg/sampler/chain.go:34-68).
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

// The same draw for long rows, spread over blocks: out[r] holds the row's first maximum (gg_argmax ran before);
// stage one sums exp(x - max) over slices of 8,192 ids (eight consecutive ids per thread), stage two finds the
// slice in which the running sum reaches the target and walks it.  The sums are float64 and their order is
// fixed (thread, warp, block, slice), though not the order of the one-block kernel above.
#define SAMP_SLICE_IDS 8192

__device__ __forceinline__ void slice_sum(const float* logits, long long ld, float temp, const int* best,
                                          double* __restrict__ zs, int V, double* dred);

__global__ void __launch_bounds__(SAMP_THREADS) sample_slice_sum_uniform_kernel(const float* logits, long long ld, float temp,
                                                                                 const int* best, double* __restrict__ zs, int V) {
    pdl_launch();
    pdl_wait();
    __shared__ double dred[33];
    slice_sum(logits, ld, temp, best, zs, V, dred);
}

__global__ void __launch_bounds__(SAMP_THREADS) sample_slice_sum_kernel(const float* logits, long long ld,
                                                                         const float* __restrict__ temps,
                                                                         const int* best, double* __restrict__ zs, int V) {
    pdl_launch();
    pdl_wait();
    __shared__ double dred[33];
    slice_sum(logits, ld, temps[blockIdx.y], best, zs, V, dred);
}

__device__ __forceinline__ void slice_sum(const float* logits, long long ld, float temp, const int* best,
                                          double* __restrict__ zs, int V, double* dred) {
    const int r = blockIdx.y, slice = blockIdx.x;
    if (temp <= 0.f) return;
    const float* x = logits + (size_t)r * ld;
    const bool scaled = temp != 1.f;
    const double inv_t = scaled ? 1.0 / (double)temp : 1.0;
    const float raw_max = x[best[r]];
    const float mx = scaled ? (float)((double)raw_max * inv_t) : raw_max;
    const int lo = slice * SAMP_SLICE_IDS + threadIdx.x * 8;
    double local = 0.0;
#pragma unroll
    for (int u = 0; u < 8; ++u) {
        const int i = lo + u;
        if (i < V) {
            const float v = scaled ? (float)((double)x[i] * inv_t) : x[i];
            local += exp((double)(v - mx));
        }
    }
    const double total = block_sum_f64(local, dred);
    if (threadIdx.x == 0) zs[(size_t)r * gridDim.x + slice] = total;
}

__global__ void __launch_bounds__(SAMP_THREADS) sample_pick_kernel(const float* logits, long long ld,
                                                                    const float* __restrict__ temps,
                                                                    const double* __restrict__ uniforms, const double* zs,
                                                                    int slices, int* out, int V) {
    pdl_launch();
    pdl_wait();
    __shared__ double pre[SAMP_THREADS];
    __shared__ double sh[3];          // 1 / Z, running sum before the slice, target
    __shared__ int sh_slice, found;
    const int r = blockIdx.x;
    const float temp = temps[r];
    if (temp <= 0.f) return;          // greedy row: out[r] already holds the first maximum
    const float* x = logits + (size_t)r * ld;
    const bool scaled = temp != 1.f;
    const double inv_t = scaled ? 1.0 / (double)temp : 1.0;
    const float raw_max = x[out[r]];
    const float mx = scaled ? (float)((double)raw_max * inv_t) : raw_max;
    __syncthreads();                  // every thread has read out[r] before it is overwritten
    if (threadIdx.x == 0) {
        double Z = 0.0;
        for (int s = 0; s < slices; ++s) Z += zs[(size_t)r * slices + s];
        const double inv = 1.0 / Z;
        double norm = 0.0;
        for (int s = 0; s < slices; ++s) norm += zs[(size_t)r * slices + s] * inv;
        const double target = uniforms[r] * norm;
        double run = 0.0;
        int pick = -1;
        for (int s = 0; s < slices; ++s) {
            const double p = zs[(size_t)r * slices + s] * inv;
            if (target - (run + p) <= 0.0) { pick = s; break; }
            run += p;
        }
        sh[0] = inv; sh[1] = run; sh[2] = target;
        sh_slice = pick;
        found = 0x7fffffff;
    }
    __syncthreads();
    const int slice = sh_slice;
    if (slice < 0) {                  // rounding left the target above the total: the last id
        if (threadIdx.x == 0) out[r] = V - 1;
        return;
    }
    const double inv = sh[0], target = sh[2];
    const int lo = slice * SAMP_SLICE_IDS + threadIdx.x * 8;
    double e[8], local = 0.0;
#pragma unroll
    for (int u = 0; u < 8; ++u) {
        const int i = lo + u;
        e[u] = 0.0;
        if (i < V) {
            const float v = scaled ? (float)((double)x[i] * inv_t) : x[i];
            e[u] = exp((double)(v - mx)) * inv;
        }
        local += e[u];
    }
    pre[threadIdx.x] = local;
    __syncthreads();
    if (threadIdx.x == 0) {
        double run = sh[1];
        for (int t = 0; t < SAMP_THREADS; ++t) { const double c = pre[t]; pre[t] = run; run += c; }
    }
    __syncthreads();
    double run = pre[threadIdx.x];
    if (run < target + 1e-300) {
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            if (lo + u < V) {
                run += e[u];
                if (target - run <= 0.0) { atomicMin(&found, lo + u); break; }
            }
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        // the slice's own sum said the target is reached inside it; if the walk's rounding disagrees, its last id
        const int last = min(V, (slice + 1) * SAMP_SLICE_IDS) - 1;
        out[r] = found == 0x7fffffff ? last : found;
    }
}

// scratch (optional): R * 128 four-byte words for the two-stage maximum, then R * ceil(V / 8192) doubles; with
// it, rows of 16,384 ids or more are spread over blocks.  Null: one block per row.
GG_API gg_sample(const float* logits, long long ld, const float* temps, const double* uniforms, int* out,
                 int R, int V, void* scratch, long long scratch_words, cudaStream_t stream) {
    if (R <= 0) return 0;
    if (V <= 0 || ld < V) return GG_ERR_ARG;
    const int slices = (V + SAMP_SLICE_IDS - 1) / SAMP_SLICE_IDS;
    const long long need = (long long)R * 128 + 2LL * R * slices;
    if (scratch == nullptr || V < 16384 || scratch_words < need || R > 65535 || (((uintptr_t)scratch) & 7)) {
        gg_launch(sample_kernel, dim3(R), dim3(SAMP_THREADS), 0, stream, 1, logits, ld, temps, uniforms, out, V);
        return gg_last_error();
    }
    int rc = gg_argmax(logits, ld, out, R, V, scratch, (long long)R * 128, stream);
    if (rc != 0) return rc;
    double* zs = reinterpret_cast<double*>(reinterpret_cast<int*>(scratch) + (size_t)R * 128);
    rc = gg_launch(sample_slice_sum_kernel, dim3(slices, R), dim3(SAMP_THREADS), 0, stream, 1, logits, ld, temps,
                   (const int*)out, zs, V);
    if (rc != 0) return rc;
    return gg_launch(sample_pick_kernel, dim3(R), dim3(SAMP_THREADS), 0, stream, 1, logits, ld, temps, uniforms,
                     (const double*)zs, slices, out, V);
}


// ----------------------------------------------------------------------------- the chain with a top-k
// (1) x = float32(float64(logit) / temp) when temp > 0 and != 1.  (2) The k largest x, ties to the lower id
// (the reference sorts, chain.go:77-103).  Value and id make one 64-bit key, larger = better and no two equal,
// so "the k best" is a threshold on that key; the k-th largest key of a set is found four bits at a time with
// per-thread counters (no atomics).  Stage one: every block holds a slice of 8,192 logits of one row in
// registers and leaves its k best keys in scratch (a row's k best are among its slices' k best).  Stage two:
// one block per row selects the k best of those and runs (3) on them, in float64 as the reference: min-p
// against the row maximum (penalties.go:35-54), softmax, top-p over the values in descending order
// (chain.go:105-133: keep until the running sum reaches p - 1e-6, the element that crosses included), and the
// draw in id order with the caller's uniform number (chain.go:135-166).  k is at most SAMP_TOPK_MAX.
#define SAMP_TOPK_MAX 1024
#define SAMP_SLICE 8192          // logits per block in stage one: eight per thread

__device__ __forceinline__ uint32_t order_key(float f) {
    // unsigned keys that order like the floats
    const uint32_t b = __float_as_uint(f);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float key_value(uint32_t key) {
    return __uint_as_float((key & 0x80000000u) ? (key & 0x7fffffffu) : ~key);
}
__device__ __forceinline__ unsigned long long best_key(float x, int id) {
    return ((unsigned long long)order_key(x) << 32) | (unsigned long long)(0xffffffffu - (uint32_t)id);
}

// The k-th largest of the keys that `key_of(j)`, j < n_mine, gives this thread (0 = no key), over the whole
// block; k >= 1.  Returns 0 when the block holds fewer than k keys (then every key is among the k best).
// Four bits per pass: every thread counts its keys per digit in sixteen 16-bit counters packed into four
// 64-bit words (so a block may hold at most 65,535 keys), a warp adds them with shuffles, lane 0 adds the
// warp's words into one of three rotating sets in shared memory, and after one barrier every thread reads
// the totals and takes the same decision.  The low 32 bits (the ids) are only walked when the k-th place
// falls among equal values.
template <typename KeyOf>
__device__ unsigned long long block_kth_largest(int n_mine, KeyOf key_of, int k, unsigned long long (*tot)[4]) {
    const int lane = threadIdx.x & 31;
    unsigned long long prefix = 0;
    int above = 0;
    if (threadIdx.x < 4) tot[0][threadIdx.x] = 0ull;
    __syncthreads();
    for (int pass = 0; pass < 16; ++pass) {
        // passes 0-7 walk the high word (the value), 8-15 the low word (the id) of keys whose value is the threshold's
        const int shift = 28 - 4 * (pass & 7);
        const uint32_t p_hi = (uint32_t)(prefix >> 32), p_lo = (uint32_t)prefix;
        const uint32_t p_word = pass < 8 ? p_hi : p_lo;
        const uint32_t mask_above = shift == 28 ? 0u : (0xffffffffu << (shift + 4));     // the digits decided in this word
        if (threadIdx.x < 4) tot[(pass + 1) % 3][threadIdx.x] = 0ull;     // last read two passes ago
        unsigned long long c4[4] = {0ull, 0ull, 0ull, 0ull};
        for (int j = 0; j < n_mine; ++j) {
            const unsigned long long key = key_of(j);
            const uint32_t hi = (uint32_t)(key >> 32), lo = (uint32_t)key;
            const uint32_t word = pass < 8 ? hi : lo;
            bool in = key != 0ull && ((word ^ p_word) & mask_above) == 0u;
            if (pass >= 8) in = in && hi == p_hi;
            const int b = (int)(word >> shift) & 15;
            const unsigned long long inc = in ? (1ull << (16 * (b & 3))) : 0ull;
#pragma unroll
            for (int q = 0; q < 4; ++q) c4[q] += (q == (b >> 2)) ? inc : 0ull;
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) c4[q] += __shfl_xor_sync(0xffffffffu, c4[q], o);
            // (two 32-bit additions: no 16-bit field overflows, so no carry crosses the halves)
            if (lane == 0 && c4[q] != 0ull) {
                uint32_t* t32 = reinterpret_cast<uint32_t*>(&tot[pass % 3][q]);
                if ((uint32_t)c4[q] != 0u) atomicAdd(t32, (uint32_t)c4[q]);
                if ((uint32_t)(c4[q] >> 32) != 0u) atomicAdd(t32 + 1, (uint32_t)(c4[q] >> 32));
            }
        }
        __syncthreads();
        int cum = above, bin = -1, at_bin = 0;
#pragma unroll
        for (int b = 15; b >= 0; --b) {
            const int t = (int)((tot[pass % 3][b >> 2] >> (16 * (b & 3))) & 0xffffull);
            if (bin < 0) {
                if (cum + t >= k) { bin = b; at_bin = t; }
                else cum += t;
            }
        }
        if (bin < 0) return 0ull;                     // fewer than k keys in the block
        prefix |= (unsigned long long)bin << (shift + (pass < 8 ? 32 : 0));
        above = cum;
        // all values decided and every key with the threshold value fits: the ids need not be walked
        if (pass == 7 && above + at_bin <= k) return prefix;
    }
    return prefix;
}

// Stage one: grid (slices, rows), 256 threads with 32 logits each (the per-pass cost of a thread is mostly fixed:
// shuffles, the barrier, the decision).  cand[(row * slices + slice) * k + j]: the slice's k best keys (0 = none).
#define SAMP_SLICE_THREADS 256
#define SAMP_SLICE_PER (SAMP_SLICE / SAMP_SLICE_THREADS)

__global__ void __launch_bounds__(SAMP_SLICE_THREADS) topk_slice_kernel(const float* logits, long long ld, int V, float temp,
                                                                        int k, unsigned long long* __restrict__ cand) {
    pdl_launch();
    pdl_wait();
    __shared__ unsigned long long tot[3][4];
    __shared__ int n_out;
    const int row = blockIdx.y, slice = blockIdx.x, tid = threadIdx.x;
    const float* x = logits + (size_t)row * ld;
    const bool scale = temp > 0.f && temp != 1.f;
    const double inv_temp = scale ? 1.0 / (double)temp : 1.0;
    unsigned long long keys[SAMP_SLICE_PER];
#pragma unroll
    for (int u = 0; u < SAMP_SLICE_PER; ++u) {
        const int i = slice * SAMP_SLICE + u * SAMP_SLICE_THREADS + tid;
        float v = i < V ? x[i] : 0.f;
        if (scale) v = (float)((double)v * inv_temp);
        keys[u] = i < V ? best_key(v, i) : 0ull;
    }
    if (tid == 0) n_out = 0;
    const unsigned long long thr = block_kth_largest(SAMP_SLICE_PER, [&](int j) { return keys[j]; }, k, tot);
    unsigned long long* dst = cand + ((size_t)row * gridDim.x + slice) * k;
    for (int j = tid; j < k; j += SAMP_SLICE_THREADS) dst[j] = 0ull;
    __syncthreads();
#pragma unroll
    for (int u = 0; u < SAMP_SLICE_PER; ++u)
        if (keys[u] != 0ull && keys[u] >= thr) dst[atomicAdd(&n_out, 1)] = keys[u];
}

// Inclusive prefix sums of one double per thread over the block, in thread order; *total gets the block's sum.
__device__ __forceinline__ double block_scan_f64(double v, double* warp_tot /* 33 */, double* total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const double y = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v += y;
    }
    __syncthreads();
    if (lane == 31) warp_tot[warp] = v;
    __syncthreads();
    if (warp == 0) {
        double t = lane < nw ? warp_tot[lane] : 0.0;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const double y = __shfl_up_sync(0xffffffffu, t, o);
            if (lane >= o) t += y;
        }
        if (lane < nw) warp_tot[lane] = t;          // inclusive over warps
        if (lane == 31) warp_tot[32] = t;
    }
    __syncthreads();
    if (warp > 0) v += warp_tot[warp - 1];
    *total = warp_tot[32];
    return v;
}

// Stage two: one block per row over its slices * k candidate keys (dynamic shared memory holds them).
// zs == null: the chain with a top-k (the softmax is over the k survivors).  zs != null: top-p and min-p without
// a top-k, for which the k survivors are only candidates: the softmax is over the whole row, whose sum
// of exp(x - max) is the sum of zs[row * z_slices ..], and flags[row] is set when the candidates do not hold
// the whole answer (min-p keeps even the last candidate, or the running sum never reaches top-p): the caller
// then takes that row through the host chain.
__global__ void __launch_bounds__(SAMP_THREADS) sample_topk_kernel(
    const unsigned long long* cand, int n_cand_keys, int top_k, float top_p, float min_p,
    const double* __restrict__ uniforms, int* __restrict__ out, const double* zs, int z_slices, int* __restrict__ flags,
    int V) {
    pdl_launch();
    pdl_wait();
    extern __shared__ unsigned long long ckeys[];
    __shared__ unsigned long long tot[3][4];
    __shared__ float cand_x[SAMP_TOPK_MAX];
    __shared__ int cand_i[SAMP_TOPK_MAX];
    __shared__ double cand_e[SAMP_TOPK_MAX];
    __shared__ int by_value[SAMP_TOPK_MAX];      // candidate slots in descending order of x (ties: lower id)
    __shared__ int by_id[SAMP_TOPK_MAX];         // candidate slots in ascending order of id
    __shared__ unsigned char keep[SAMP_TOPK_MAX];
    __shared__ int n_sel, pick_r, last_r;
    __shared__ double wtot[33], z_row;
    const int row = blockIdx.x, tid = threadIdx.x;
    const unsigned long long* src = cand + (size_t)row * n_cand_keys;
    for (int j = tid; j < n_cand_keys; j += SAMP_THREADS) ckeys[j] = src[j];
    if (tid == 0) n_sel = 0;
    __syncthreads();
    const int mine = (n_cand_keys - tid + SAMP_THREADS - 1) / SAMP_THREADS;
    const unsigned long long thr = block_kth_largest(mine, [&](int j) { return ckeys[tid + j * SAMP_THREADS]; }, top_k, tot);
    for (int j = tid; j < n_cand_keys; j += SAMP_THREADS) {
        const unsigned long long key = ckeys[j];
        if (key != 0ull && key >= thr) {
            const int s = atomicAdd(&n_sel, 1);
            cand_x[s] = key_value((uint32_t)(key >> 32));
            cand_i[s] = (int)(0xffffffffu - (uint32_t)key);
        }
    }
    __syncthreads();
    const int n = n_sel;                          // min(top_k, V)
    // ---- orders: by value (descending, ties to the lower id) and by id, by counting
    for (int a = tid; a < n; a += SAMP_THREADS) {
        const float xa = cand_x[a];
        const int ia = cand_i[a];
        int rv = 0, ri = 0;
        for (int b = 0; b < n; ++b) {
            const float xb = cand_x[b];
            const int ib = cand_i[b];
            rv += (xb > xa) || (xb == xa && ib < ia);
            ri += ib < ia;
        }
        by_value[rv] = a;
        by_id[ri] = a;
    }
    __syncthreads();
    const float xmax = cand_x[by_value[0]];
    // ---- min-p and the exponentials (the maximum of the whole row is among the candidates)
    for (int a = tid; a < n; a += SAMP_THREADS) {
        const double e = exp((double)(cand_x[a] - xmax));
        const bool ok = !(min_p > 0.f && e < (double)min_p);     // p < min_p * p_max with p_max = e(0) / Z
        keep[a] = ok ? 1 : 0;
        cand_e[a] = ok ? e : 0.0;
    }
    __syncthreads();
    // ---- the softmax's denominator: over the survivors, or over the whole row
    double Z;
    {
        const double mine = tid < n ? cand_e[by_id[tid]] : 0.0;
        double total;
        block_scan_f64(mine, wtot, &total);
        // (min-p masks before the softmax, so with it the denominator is the sum over its survivors, all of
        // which are candidates unless the row gets flagged)
        if (zs != nullptr && !(min_p > 0.f)) {
            if (tid == 0) {
                double z = 0.0;
                for (int sl = 0; sl < z_slices; ++sl) z += zs[(size_t)row * z_slices + sl];
                z_row = z;
            }
            __syncthreads();
            total = z_row;
        }
        Z = total;
    }
    bool incomplete = false;
    if (zs != nullptr && n < V && min_p > 0.f && keep[by_value[n - 1]]) incomplete = true;      // min-p may keep more
    // ---- top-p: in descending order keep until the running sum reaches p - 1e-6, the crossing element included
    if (top_p > 0.f && top_p < 1.f) {
        const double thr_p = (double)top_p - 1e-6;
        const int a = tid < n ? by_value[tid] : 0;
        const double p = (tid < n && keep[a]) ? cand_e[a] / Z : 0.0;
        double total;
        const double cum = block_scan_f64(p, wtot, &total);
        if (tid < n && keep[a] && cum - p >= thr_p) keep[a] = 0;
        if (zs != nullptr && n < V && total < thr_p) incomplete = true;                           // the nucleus goes on
    }
    if (tid == 0) { pick_r = 0x7fffffff; last_r = -1; }
    __syncthreads();
    // ---- the draw in id order
    {
        const int a = tid < n ? by_id[tid] : 0;
        const bool kept = tid < n && keep[a];
        const double p = kept ? cand_e[a] / Z : 0.0;
        double total;
        const double run = block_scan_f64(p, wtot, &total);
        const double target = uniforms[row] * total;
        if (kept) {
            atomicMax(&last_r, tid);
            if (target - run <= 0.0) atomicMin(&pick_r, tid);
        }
        __syncthreads();
        if (tid == 0) {
            int pick;
            if (total > 0.0) pick = cand_i[by_id[pick_r != 0x7fffffff ? pick_r : last_r]];
            else pick = cand_i[by_value[0]];
            out[row] = pick;
            if (flags != nullptr) flags[row] = incomplete ? 1 : 0;
        }
    }
}

// Scratch that gg_sample_topk needs for R rows of V logits with this top-k, in 64-bit words.
GG_API gg_sample_topk_scratch_words(int R, int V, int top_k, long long* words) {
    if (R <= 0 || V <= 0 || top_k < 1 || words == nullptr) return GG_ERR_ARG;
    const int k = top_k < V ? top_k : V;
    const long long slices = (V + SAMP_SLICE - 1) / SAMP_SLICE;
    *words = (long long)R * slices * k;
    return 0;
}

// out[r] = the reference's sampling chain on row r with a top-k (1 <= min(top_k, V) <= 1024).  temp <= 0 or
// == 1: no scaling; top_p outside (0, 1) and min_p <= 0: off.  uniforms[r] in [0, 1).  scratch: what
// gg_sample_topk_scratch_words says.
GG_API gg_sample_topk(const float* logits, long long ld, float temp, int top_k, float top_p, float min_p,
                      const double* uniforms, int* out, int R, int V, void* scratch, long long scratch_words,
                      cudaStream_t stream) {
    if (R <= 0) return 0;
    if (V <= 0 || ld < V || top_k < 1 || R > 65535) return GG_ERR_ARG;
    const int k = top_k < V ? top_k : V;
    const int slices = (V + SAMP_SLICE - 1) / SAMP_SLICE;
    const long long per_row = (long long)slices * k;
    if (k > SAMP_TOPK_MAX || scratch == nullptr || scratch_words < per_row * R) return GG_ERR_ARG;
    const size_t smem = (size_t)per_row * sizeof(unsigned long long);
    if (smem > 160 * 1024) return GG_ERR_ARG;          // 1,024 best of 20 slices still fit
    static size_t configured = 0;
    if (smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(sample_topk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = smem;
    }
    int rc = gg_launch(topk_slice_kernel, dim3(slices, R), dim3(SAMP_SLICE_THREADS), 0, stream, 1, logits, ld, V, temp, k,
                       (unsigned long long*)scratch);
    if (rc != 0) return rc;
    return gg_launch(sample_topk_kernel, dim3(R), dim3(SAMP_THREADS), smem, stream, 1,
                     (const unsigned long long*)scratch, (int)per_row, k, top_p, min_p, uniforms, out,
                     (const double*)nullptr, 0, (int*)nullptr, V);
}

// Top-p and / or min-p without a top-k (temp > 0): the 1,024 largest logits of each row are the candidates, the
// softmax runs over the whole row, and flags[r] = 1 says that row r's answer may lie beyond the candidates
// (out[r] is then not to be used).  scratch: R * 128 four-byte words, then R * ceil(V / 8192) doubles, then
// R * ceil(V / 8192) * min(V, 1024) 64-bit words; all of it 8-byte aligned.
GG_API gg_sample_nucleus(const float* logits, long long ld, float temp, float top_p, float min_p, const double* uniforms,
                         int* out, int* flags, int R, int V, void* scratch, long long scratch_bytes, cudaStream_t stream) {
    if (R <= 0) return 0;
    if (V <= 0 || ld < V || R > 65535 || !(temp > 0.f) || flags == nullptr || scratch == nullptr || (((uintptr_t)scratch) & 7))
        return GG_ERR_ARG;
    const int k = V < SAMP_TOPK_MAX ? V : SAMP_TOPK_MAX;
    const int slices = (V + SAMP_SLICE - 1) / SAMP_SLICE;
    const long long per_row = (long long)slices * k;
    const long long need = (long long)R * 128 * 4 + (long long)R * slices * 8 + per_row * R * 8;
    if (scratch_bytes < need) return GG_ERR_ARG;
    const size_t smem = (size_t)per_row * sizeof(unsigned long long);
    if (smem > 160 * 1024) return GG_ERR_ARG;
    static size_t configured = 0;
    if (smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(sample_topk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = smem;
    }
    int* best = out;                                   // the row maxima's ids, overwritten by the samples at the end
    double* zs = reinterpret_cast<double*>(reinterpret_cast<int*>(scratch) + (size_t)R * 128);
    unsigned long long* cand = reinterpret_cast<unsigned long long*>(zs + (size_t)R * slices);
    int rc = gg_argmax(logits, ld, best, R, V, scratch, (long long)R * 128, stream);
    if (rc != 0) return rc;
    // every row at this temperature: the slice sums take one temperature per row
    rc = gg_launch(sample_slice_sum_uniform_kernel, dim3(slices, R), dim3(SAMP_THREADS), 0, stream, 1, logits, ld, temp,
                   (const int*)best, zs, V);
    if (rc != 0) return rc;
    rc = gg_launch(topk_slice_kernel, dim3(slices, R), dim3(SAMP_SLICE_THREADS), 0, stream, 1, logits, ld, V, temp, k, cand);
    if (rc != 0) return rc;
    return gg_launch(sample_topk_kernel, dim3(R), dim3(SAMP_THREADS), smem, stream, 1, (const unsigned long long*)cand,
                     (int)per_row, k, top_p, min_p, uniforms, out, (const double*)zs, slices, flags, V);
}



// ----------------------------------------------------------------------------- repeat penalty on the device
// The last `last_n` ids of each sequence (prompt and generated) live in a ring per sequence:
// hist[ring_row][last_n], hist_len[ring_row] ids valid (at most last_n), hist_pos[ring_row] the slot the next
// id goes to.  Before sampling, every distinct id of the ring is penalised once: logit > 0 ? logit / penalty
// : logit * penalty (pkg/sampler/penalties.go:5-32); after sampling, the new id is appended, so that the
// next step, which may already be queued, sees it without the host.
__global__ void repeat_penalty_kernel(float* logits, long long ld, int V, const int* __restrict__ hist,
                                      const int* __restrict__ hist_len, const int* __restrict__ ring_rows, int last_n,
                                      float penalty) {
    pdl_launch();
    pdl_wait();
    const int r = blockIdx.x;
    const int* h = hist + (size_t)ring_rows[r] * last_n;
    const int n = hist_len[ring_rows[r]];
    float* x = logits + (size_t)r * ld;
    for (int t = threadIdx.x; t < n; t += blockDim.x) {
        const int id = h[t];
        if (id < 0 || id >= V) continue;
        bool first = true;                       // each distinct id once: the lowest slot that holds it acts
        for (int u = 0; u < t; ++u) first = first && (h[u] != id);
        if (first) {
            const float v = x[id];
            x[id] = v > 0.f ? v / penalty : v * penalty;
        }
    }
}

__global__ void history_append_kernel(const int* tokens, const int* __restrict__ ring_rows, int* hist, int* hist_len,
                                      int* hist_pos, int last_n, int rows) {
    pdl_launch();
    pdl_wait();
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= rows) return;
    const int row = ring_rows[r];
    const int p = hist_pos[row];
    hist[(size_t)row * last_n + p] = tokens[r];
    hist_pos[row] = p + 1 == last_n ? 0 : p + 1;
    if (hist_len[row] < last_n) hist_len[row] += 1;
}

GG_API gg_repeat_penalty(float* logits, long long ld, int R, int V, const int* hist, const int* hist_len,
                         const int* ring_rows, int last_n, float penalty, cudaStream_t stream) {
    if (R <= 0) return 0;
    if (V <= 0 || ld < V || last_n <= 0 || !(penalty > 0.f)) return GG_ERR_ARG;
    gg_launch(repeat_penalty_kernel, dim3(R), dim3(128), 0, stream, 1, logits, ld, V, hist, hist_len, ring_rows, last_n, penalty);
    return gg_last_error();
}

GG_API gg_history_append(const int* tokens, const int* ring_rows, int* hist, int* hist_len, int* hist_pos, int last_n,
                         int R, cudaStream_t stream) {
    if (R <= 0) return 0;
    if (last_n <= 0) return GG_ERR_ARG;
    gg_launch(history_append_kernel, dim3((R + 127) / 128), dim3(128), 0, stream, 1, tokens, ring_rows, hist, hist_len,
              hist_pos, last_n, R);
    return gg_last_error();
}
