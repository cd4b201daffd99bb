/* gg_gemm_tc_static: the tensor-core product for callers that must not allocate.
 *
 * This entry point has no counterpart in the reference (magomedcoder/gogguf); it is an addition of
 * this library.
 *
 * Who needs it: code that runs where the CUDA allocator is off limits - a plug-in inside a host
 * program that owns all device memory and forbids cudaMalloc in its callbacks, a real-time loop
 * that may not take the allocator's locks or its implicit synchronisation, a process that has
 * handed its whole memory budget to a pool.  The regular entry point, gg_gemm_tc, needs a float32
 * scratch buffer from its caller whenever it splits the K dimension (small batches); such callers
 * have nowhere to get one.  (gg_gemm_tc also has a form that adds its partial sums inside
 * thread-block clusters and needs no scratch; this entry point is the scratch form, whose split of K
 * may be finer and which does not depend on cluster launches.)
 *
 * What it does instead: the scratch lives in a file-scope `static __device__` array inside the
 * library, GG_STATIC_SCRATCH_FLOATS floats (16 MiB).  Every GPU on which the library is loaded
 * holds that array from load until the process exits.  The function computes
 *     out[M, N] (mode) = x[M, K] * w[N, K]^T      (bfloat16 operands, float32 accumulation)
 * exactly as gg_gemm_tc's scratch form (use_cluster = 0) does, with the same kernels and the same
 * split of K, so results are bit-identical to it.  The caller passes inputs, the output and the status word; the
 * function calls no cudaMalloc, cudaFree or any other allocating routine.
 *
 * Limits and rules:
 *   - splits * M * N (splits as gg_gemm_tc_splits(M, N, K, 0) reports) must not exceed
 *     GG_STATIC_SCRATCH_FLOATS; larger products are refused with status -1 before anything is
 *     launched.  Products that need no split (M > 128, or few K slabs) never touch the array.
 *   - The first call on a device looks up the array's device address (cudaGetSymbolAddress, with
 *     that device current).  The kernels' shared-memory attribute is set once per process, by the
 *     first call of all (this library drives one GPU; a process that uses it on a second device
 *     should call once there as well and check the return code).  Make these first calls outside
 *     any stream capture.
 *   - All calls share the one array, and it keeps what the last call left in it.  Nothing in it has
 *     to start at zero: a call reads back only elements that the same call has just written.  Two
 *     calls that may overlap on the GPU (different streams without an ordering between them) race
 *     on the array; put them on one stream or order them with events.
 *
 * Arguments as gg_gemm_tc: out_mode 0 = bfloat16 store, 1 = float32 store, 2 = float32 add;
 * ldx / ldo are row strides in elements; status points to one zero-initialised int on the device.
 * Returns 0, a negative refusal code, or a cudaError_t.
 */
#pragma once
#include <cuda_runtime.h>

#define GG_STATIC_SCRATCH_FLOATS (4 * 1024 * 1024)

#ifdef __cplusplus
extern "C"
#endif
int gg_gemm_tc_static(const void* x, const void* w, void* out, int out_mode, int M, int N, int K,
                      long long ldx, long long ldo, int* status, cudaStream_t stream);
