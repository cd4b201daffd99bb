// gg_gemm_tc_static: gg_gemm_tc with its split-K scratch in a static device array, for callers
// that cannot allocate.  See gemm_tcgen05_static.h for who needs this and for the rules.
// Not in the reference; an addition of this library.
//
// The kernels are those of gemm_tcgen05.cu, compiled into this library a second time by including
// that file, so the two entry points run the same code and give the same bits.
#include "gemm_tcgen05.cu"
#include "gemm_tcgen05_static.h"

#include <mutex>

// The scratch.  In host code this name is only a handle: its device address must be asked for
// (cudaGetSymbolAddress) before it can be given to a kernel.
static __device__ __align__(256) float gg_static_scratch[GG_STATIC_SCRATCH_FLOATS];

namespace {
constexpr int MAX_DEVICES = 64;
float* scratch_address[MAX_DEVICES] = {nullptr};
std::mutex setup_lock;

// Once per device, with that device current: the device address of the array.
int static_scratch(float** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= MAX_DEVICES) return GG_ERR_ARG;
    std::lock_guard<std::mutex> hold(setup_lock);
    if (scratch_address[dev] == nullptr) {
        float* p = nullptr;
        e = cudaGetSymbolAddress((void**)&p, gg_static_scratch);
        if (e != cudaSuccess) return (int)e;
        if (p == nullptr) return GG_ERR_ARG;
        scratch_address[dev] = p;
    }
    *out = scratch_address[dev];
    return 0;
}
}  // namespace

GG_API gg_gemm_tc_static(const void* x, const void* w, void* out, int out_mode, int M, int N, int K,
                         long long ldx, long long ldo, int* status, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    const int splits = gg_gemm_tc_splits(M, N, K, 0);     // the scratch form, not the cluster form
    if (splits <= 0) return GG_ERR_ARG;
    float* scratch = nullptr;
    long long need = 0;
    if (splits > 1) {
        need = (long long)splits * M * N;
        if (need > (long long)GG_STATIC_SCRATCH_FLOATS) return GG_ERR_ARG;   // beyond the stated maximum
        const int rc = static_scratch(&scratch);
        if (rc != 0) return rc;
    }
    return gg_gemm_tc(x, w, out, out_mode, M, N, K, ldx, ldo, scratch, need, 0, status, stream);
}
