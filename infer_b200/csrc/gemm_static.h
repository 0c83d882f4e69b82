// ib_gemm_tc_static: the tensor-core matrix product for callers that must not allocate.
//
// This entry point has no counterpart in the reference engine (RyanXiaoo/infer): it is an addition of this library.
//
// Who it is for. Some code that wants out = x . w^T (+ bias) (+ residual) cannot call cudaMalloc, or anything that
// might: a serving loop whose memory is budgeted to the last byte at start-up (weights, page pools) and which treats
// any later allocation as a fault; code that runs between the steps of a latency-critical loop, where cudaMalloc's
// implicit device synchronisation would stall every stream; an embedder that reaches this library through its C ABI
// from a process whose device memory belongs to another allocator. The regular entry point, ib_gemm_tc, leaves the
// split-K scratch (partial tiles and per-tile counters) to its caller; this one brings its own.
//
// How. The scratch lives in one file-scope `static __device__ __align__(256)` array of IB_GEMM_STATIC_SCRATCH_BYTES
// (8 MiB) inside the library image: every GPU that loads the library holds those 8 MiB until the process exits,
// whether the entry point is ever called or not. The first call on a device looks the array's device address up
// (cudaGetSymbolAddress, with that device current) and keeps it; make that first call outside of any stream capture.
// No call allocates or frees: no cudaMalloc, cudaFree, or allocating library routine.
//
// Limits and rules.
//  - Only a plan that adds its K slices through global memory uses the array (ib_gemm_tc_plan states how many floats
//    and counters that takes): products of more than 128 rows with very few output tiles. If such a plan needs more
//    than the array holds, the call is refused with an error and nothing runs. Every other plan (no split, or slices
//    that meet in a thread-block cluster's shared memory) is given no scratch at all and always fits.
//  - Every call on a device shares the one array. Calls that are ordered (same stream, or otherwise serialised) are
//    fine; calls that overlap on the GPU race on the scratch and give wrong sums. The array keeps the last call's
//    partial tiles; the counters at its start are zeroed on the stream before each launch.
//  - Inputs and outputs are the caller's, exactly as for ib_gemm_tc: x [M, K] and w [N, K] bfloat16 with 16-byte
//    aligned bases and K a multiple of 8; bias float [N] or null; residual float [M, N] or null (may alias out);
//    out float or bfloat16 [M, N]; status: one int in device memory that a kernel raises when a bounded wait ran out.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#define IB_GEMM_STATIC_SCRATCH_BYTES (8u << 20)

#ifdef __cplusplus
extern "C" {
#endif

// Returns 0, or a negative code (see ib_last_error() of the same library for the text).
// out_dtype: 0 = float, 1 = bfloat16. sm_count: SMs of the device (used to plan the split); 0 = assume 148.
int ib_gemm_tc_static(const void* x, const void* w, const float* bias, const float* residual, void* out, int64_t M,
                      int64_t N, int64_t K, int out_dtype, int sm_count, int* status, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
