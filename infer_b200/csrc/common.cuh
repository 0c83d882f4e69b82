// Shared helpers of the sm_100a kernels: storage types, error reporting, warp/block reductions.
//
// Every launcher in this library is an extern "C" function that takes raw device pointers, sizes
// and a CUDA stream, enqueues its work without synchronising, and returns 0 or an error code.
// After a non-zero return, ib_last_error() (one copy per shared library) describes the problem.
// Launchers refuse sizes they cannot handle (return IB_ERR_ARG) instead of computing something else.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cstdint>
#include <cstdio>
#include <cstdarg>

#define IB_OK 0
#define IB_ERR_ARG -1      // a size, dtype or pointer the kernel does not accept
#define IB_ERR_CUDA -2     // the CUDA runtime reported an error at launch
#define IB_ERR_DEVICE -3   // a kernel reported a failure through its status word

#define IB_F32 0
#define IB_BF16 1

namespace ib {

inline char* error_buffer() {
    static thread_local char buf[512];
    return buf;
}

inline int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(error_buffer(), 512, fmt, ap);
    va_end(ap);
    return code;
}

inline int check_launch(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(IB_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
    return IB_OK;
}

// ---------------------------------------------------------------------------------------------------------------
// Programmatic dependent launch. Every kernel of this library is launched with the "programmatic stream
// serialization" attribute: it may be scheduled while its predecessor in the stream is still draining, and runs its
// own set-up (and, in the streaming kernels, its first weight loads, which no predecessor writes) before pdl_wait(),
// which returns once every predecessor grid has completed and its writes are visible. A kernel therefore touches
// nothing that a predecessor may read or write before pdl_wait(). pdl_launch_dependents() lets the successor be
// scheduled once all CTAs of this grid have passed it; a kernel that never calls it releases the successor at exit.
// Inside a captured CUDA graph the attribute becomes a programmatic edge between the kernel nodes.
inline bool& pdl_enabled() {
    static bool enabled = true;
    return enabled;
}

template <typename... KArgs, typename... Args>
inline int launch(const char* what, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                  unsigned cluster_x, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attrs[2];
    unsigned n = 0;
    if (pdl_enabled()) {
        attrs[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attrs[n].val.programmaticStreamSerializationAllowed = 1;
        n++;
    }
    if (cluster_x > 1) {
        attrs[n].id = cudaLaunchAttributeClusterDimension;
        attrs[n].val.clusterDim.x = cluster_x;
        attrs[n].val.clusterDim.y = 1;
        attrs[n].val.clusterDim.z = 1;
        n++;
    }
    cfg.attrs = attrs;
    cfg.numAttrs = n;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
    if (e != cudaSuccess) return fail(IB_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
    return IB_OK;
}

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Asks the memory system to bring `bytes` (a multiple of 16) at `base` into L2, this CTA taking its share of the
// range. Used by decode kernels to fetch the weights of a kernel that runs later, while they themselves are bound by
// latency and leave HBM idle. A hint: nothing waits for it and nothing breaks if the lines are evicted again.
__device__ __forceinline__ void l2_prefetch_share(const void* base, int64_t bytes, int cta, int n_cta) {
    if (!base || bytes <= 0) return;
    constexpr int64_t PIECE = 4096;
    const int64_t per = (((bytes + n_cta - 1) / n_cta) + PIECE - 1) / PIECE * PIECE;
    const int64_t lo = int64_t(cta) * per, hi = lo + per < bytes ? lo + per : bytes;
    const char* b = static_cast<const char*>(base);
    for (int64_t off = lo + int64_t(threadIdx.x) * PIECE; off < hi; off += int64_t(blockDim.x) * PIECE) {
        const uint32_t n = uint32_t(hi - off < PIECE ? hi - off : PIECE) & ~15u;
        if (n) asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(b + off), "r"(n) : "memory");
    }
}

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

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

// Block-wide sum / max for blocks of up to 1024 threads (a multiple of 32). `red` is 32 floats of
// shared memory. The order of additions depends only on the block size, so results do not depend
// on what else runs. All threads get the result.
__device__ __forceinline__ float block_sum(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float t = lane < nw ? red[lane] : 0.0f;
    return warp_sum(t);
}

__device__ __forceinline__ float block_max(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float t = lane < nw ? red[lane] : -INFINITY;
    return warp_max(t);
}

}  // namespace ib

#define IB_EXPORT extern "C" __attribute__((visibility("default")))

#define IB_DEFINE_LAST_ERROR() \
    IB_EXPORT const char* ib_last_error() { return ib::error_buffer(); } \
    IB_EXPORT void ib_set_pdl(int on) { ib::pdl_enabled() = on != 0; }
