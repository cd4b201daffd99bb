// Self-checks of the helpers that the kernels' fault handling rests on, small enough to run in a test.
//
// wait_probe_kernel: one CTA waits, with the package's own bounded wait (tma::mbar_wait_for), on an mbarrier
// that nothing ever arrives at.  No TMA copy, no tensor memory, nothing else in flight: the wait can only run
// out.  It must then return false, leave its code in the status word, raise the CTA's abort flag, and a second
// role waiting on the same flag must give up as well, so that the kernel ends by itself after about
// `limit_cycles` clock cycles.  This is the path every kernel with a ring of stages takes when a copy never
// lands; in normal operation it never runs.
#include "common.cuh"
#include "tma_util.cuh"

namespace {

__global__ void __launch_bounds__(64) wait_probe_kernel(long long limit_cycles, int code, int* status, int* report) {
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        tma::mbar_init(&bar, 1);
        abort_flag = 0;
        tma::mbar_fence_init();
    }
    __syncthreads();
    const long long t0 = clock64();
    bool ok = true;
    if (threadIdx.x == 0) {
        // the role whose wait runs out
        ok = tma::mbar_wait_for(&bar, 0, &abort_flag, status, code, limit_cycles);
        report[0] = ok ? 1 : 0;
        report[2] = (int)((clock64() - t0) >> 10);               // elapsed, in units of 1024 cycles
    } else if (threadIdx.x == 32) {
        // a second role with a far longer limit of its own: it must leave because of the abort flag
        ok = tma::mbar_wait_for(&bar, 0, &abort_flag, status, code + 1, limit_cycles * 1000);
        report[1] = ok ? 1 : 0;
        report[3] = (int)((clock64() - t0) >> 10);
    }
    __syncthreads();
    if (threadIdx.x == 0) report[4] = abort_flag;
}

}  // namespace

// report: 5 ints on the device: [0] wait returned true (1) or false (0); [1] the same for the second role;
// [2], [3] their elapsed clock cycles / 1024; [4] the abort flag at the end.  limit_cycles is bounded to about a
// tenth of a second so that the probe can never hold a GPU.
GG_API gg_wait_probe(long long limit_cycles, int code, int* status, int* report, cudaStream_t stream) {
    if (limit_cycles <= 0 || limit_cycles > 200000000LL || status == nullptr || report == nullptr) return GG_ERR_ARG;
    wait_probe_kernel<<<1, 64, 0, stream>>>(limit_cycles, code, status, report);
    return gg_last_error();
}
