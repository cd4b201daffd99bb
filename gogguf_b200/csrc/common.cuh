// Shared helpers for the sm_100a kernels of gogguf_b200.
//
// Conventions of every launcher (functions marked GG_API):
//   * plain C linkage, int status: 0 ok, a positive value is a cudaError_t,
//     negative values are refusals (-1 size/argument, -2 dtype combination).
//   * dtype codes: 0 = float32, 1 = bfloat16.
//   * all pointers are device pointers; the last argument is the stream.
//   * nothing is allocated; scratch is passed in by the caller.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

#define GG_API extern "C" __attribute__((visibility("default"))) int

#define GG_F32 0
#define GG_BF16 1

#define GG_ERR_ARG (-1)
#define GG_ERR_DTYPE (-2)
#define GG_ERR_DEVICE (-3)
#define GG_ERR_TIMEOUT (-4)
#define GG_ERR_TMAP (-5)

typedef __nv_bfloat16 bf16;

static inline int gg_last_error() { return (int)cudaGetLastError(); }

template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<bf16>(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f<bf16>(float v) { return __float2bfloat16_rn(v); }

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

// Sum over a block of up to 1024 threads; every thread gets the result.  The
// order of the additions depends only on the block size, never on the data or
// on what else runs, so results are reproducible.
__device__ __forceinline__ float block_sum(float v, float* red /* >= 33 floats of shared memory */) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarps ? red[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}

// Dispatch helpers: call `expr` with `T` bound to the type of a dtype code.
#define GG_DISPATCH_DTYPE(code, T, ...)                       \
    do {                                                      \
        if ((code) == GG_F32) { typedef float T; __VA_ARGS__; } \
        else if ((code) == GG_BF16) { typedef bf16 T; __VA_ARGS__; } \
        else return GG_ERR_DTYPE;                             \
    } while (0)

// ----------------------------------------------------------------------------- checked page tables
// The debug build (-DGG_DEBUG_BOUNDS; GOGGUF_B200_DEBUG=1 selects it) makes every kernel that follows a page
// table check the index into the table and the page id it finds there before it uses them.  A bad one is
// recorded in the status word (code 41-48 names the kernel) and page 0 is read instead, so the kernel never
// touches memory outside the pools; the host raises when it next checks the status word.  In the normal
// build gg_page() is the plain table read.  It stands in for a memory checker, which cannot run here.
struct PageBounds {
    int n_pages;         // pages in the pool
    int* status;         // the device's status word (may be null: nothing is recorded)
};
__device__ __forceinline__ int gg_page(const int* pt, int idx, int max_pages, const PageBounds& pb, int code) {
#ifdef GG_DEBUG_BOUNDS
    if (idx < 0 || idx >= max_pages) {
        if (pb.status != nullptr) atomicCAS(pb.status, 0, code);
        return 0;
    }
    const int page = pt[idx];
    if (page < 0 || page >= pb.n_pages) {
        if (pb.status != nullptr) atomicCAS(pb.status, 0, code);
        return 0;
    }
    return page;
#else
    return pt[idx];
#endif
}
// The same for a kernel that WRITES through the table (the cache writers): a bad index or page id is recorded
// (codes 46-48) and -1 comes back, on which the caller writes nothing.  In the normal build: the plain read.
__device__ __forceinline__ int gg_page_w(const int* pt, int idx, int max_pages, const PageBounds& pb, int code) {
#ifdef GG_DEBUG_BOUNDS
    const int page = (idx < 0 || idx >= max_pages) ? -1 : pt[idx];
    if (page < 0 || page >= pb.n_pages) {
        if (pb.status != nullptr) atomicCAS(pb.status, 0, code);
        return -1;
    }
    return page;
#else
    return pt[idx];
#endif
}
static inline int gg_debug_bounds() {
#ifdef GG_DEBUG_BOUNDS
    return 1;
#else
    return 0;
#endif
}

// ----------------------------------------------------------------------------- dependent launches
// Kernels of a step are launched with programmatic stream serialisation: a kernel may become
// resident while its predecessor in the stream is still draining, run its prologue (barrier set-up,
// tensor-memory allocation, loads of weights, which no kernel writes), and must call pdl_wait()
// before it touches anything a predecessor reads or writes.  Every kernel calls pdl_wait(), so
// "my predecessor has completed" holds transitively for all earlier kernels.  pdl_launch() lets the
// successor start early.  Without the launch attribute both are no-ops.
//
// One rule came out of a stall seen on B200: a kernel that runs in many waves of CTAs and whose
// CTAs cannot share an SM with the CTAs of the kernel after it (both need most of the shared
// memory) does NOT call pdl_launch().  With the early release, the persistent product that follows
// prefill attention took over SMs as they came free while attention CTAs were still waiting to be
// scheduled, and the two kernels waited for each other; the cause was not established (reading the
// two kernels again found no wait of one on the other: they never share an SM, so not tensor memory;
// the pair's cluster barriers and the dependency wait need nothing an attention CTA holds), so such
// kernels simply release their successor by completing.  Decode attention releases at its top only
// when its whole grid is resident at once, and after its pages otherwise.  Light kernels with many
// CTAs (norms, rotary) share SMs with whatever follows and keep the early release.
//
// A second rule, for the compiler: a pointer to data that an earlier kernel of the same step writes
// (activations, the residual stream, q, the cache, rotary tables, logits, partial results) is never
// declared `const ... __restrict__`.  Loads through such a pointer are invariant loads (ld.global.nc)
// that the compiler may move above griddepcontrol.wait, "memory" clobber or not; that happened to the
// q loads of decode attention, which then read the previous layer's q.  Weights and the step's integer
// inputs (copied to the device before the step's first kernel) do not change while a step runs and
// keep the qualifier.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

#include <cstdlib>
static inline bool gg_pdl_enabled() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("GOGGUF_B200_PDL");
        v = (e != nullptr && e[0] == '0') ? 0 : 1;
    }
    return v == 1;
}

// Launch `kernel` with the dependent-launch attribute and, when cluster_z > 1, clusters of (1, 1, cluster_z).
template <typename... KArgs, typename... Args>
static inline int gg_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                            int cluster_z, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int n = 0;
    if (gg_pdl_enabled()) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    if (cluster_z > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = 1;
        attr[n].val.clusterDim.y = 1;
        attr[n].val.clusterDim.z = (unsigned)cluster_z;
        ++n;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
    if (e != cudaSuccess) return (int)e;
    return (int)cudaGetLastError();
}

// As gg_launch, with clusters of (2, 1, 1): pairs of CTAs with consecutive blockIdx.x.
template <typename... KArgs, typename... Args>
static inline int gg_launch2(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                             Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int n = 0;
    if (gg_pdl_enabled()) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = 2;
    attr[n].val.clusterDim.y = 1;
    attr[n].val.clusterDim.z = 1;
    ++n;
    cfg.attrs = attr;
    cfg.numAttrs = n;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
    if (e != cudaSuccess) return (int)e;
    return (int)cudaGetLastError();
}
