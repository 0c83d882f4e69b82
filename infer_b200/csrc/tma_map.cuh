// Tensor maps (TMA descriptors) of row-major bfloat16 matrices, shared by the kernels that load tiles with
// cp.async.bulk.tensor: boxes of box_rows x 64 elements (one 128-byte swizzle line per row), zero fill outside.
#pragma once
#include "common.cuh"

#include <cuda.h>
#include <mutex>
#include <unordered_map>

namespace ib {

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeFn encode_fn() {
    static EncodeFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeFn>(ptr);
    });
    return fn;
}

struct MapKey {
    const void* ptr; int64_t rows, cols; int box_rows;
    bool operator==(const MapKey& o) const { return ptr == o.ptr && rows == o.rows && cols == o.cols && box_rows == o.box_rows; }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        size_t h = std::hash<const void*>()(k.ptr);
        h ^= std::hash<int64_t>()(k.rows * 1315423911LL + k.cols * 2654435761LL + k.box_rows) + 0x9e3779b97f4a7c15ULL + (h << 6) + (h >> 2);
        return h;
    }
};

// Tensor map of a row-major bf16 matrix [rows, cols] with boxes of box_rows x 64 elements, 128-byte swizzle,
// zero fill outside. Encoding is pure host arithmetic on (pointer, shape); results are cached.
inline int get_map(const void* ptr, int64_t rows, int64_t cols, int box_rows, CUtensorMap* out) {
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
    static std::mutex mu;
    const MapKey key{ptr, rows, cols, box_rows};
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it != cache.end()) { *out = it->second; return IB_OK; }
    EncodeFn fn = encode_fn();
    if (!fn) return ib::fail(IB_ERR_CUDA, "tensor map: cuTensorMapEncodeTiled is not available from this driver");
    const cuuint64_t dims[2] = {cuuint64_t(cols), cuuint64_t(rows)};
    const cuuint64_t strides[1] = {cuuint64_t(cols) * 2};
    const cuuint32_t box[2] = {64u, cuuint32_t(box_rows)};
    const cuuint32_t estr[2] = {1, 1};
    CUtensorMap m;
    const CUresult r = fn(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return ib::fail(IB_ERR_CUDA, "tensor map: cuTensorMapEncodeTiled failed with code %d", int(r));
    if (cache.size() > 8192) cache.clear();
    cache.emplace(key, m);
    *out = m;
    return IB_OK;
}

}  // namespace ib
