// Tensor maps (TMA descriptors) over row-major bfloat16 matrices, made through
// the driver's cuTensorMapEncodeTiled (looked up at run time, so the libraries do
// not link against the driver) and kept in a small cache.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <mutex>
#include <unordered_map>

namespace chibi {

constexpr int TENSOR_MAP_BOX_COLS = 64;   // bf16 per row of a box = one 128-byte swizzle atom

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled()
{
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess
            && q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    });
    return fn;
}

struct MapKey {
    const void* ptr;
    long long rows, cols, stride;
    int box_rows;
    bool operator==(const MapKey& o) const
    {
        return ptr == o.ptr && rows == o.rows && cols == o.cols && stride == o.stride && box_rows == o.box_rows;
    }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const
    {
        size_t h = reinterpret_cast<size_t>(k.ptr);
        h = h * 1000003u ^ (size_t)k.rows;
        h = h * 1000003u ^ (size_t)k.cols;
        h = h * 1000003u ^ (size_t)k.stride;
        h = h * 1000003u ^ (size_t)k.box_rows;
        return h;
    }
};

// A map over a row-major bf16 matrix [rows, cols] with `stride` elements between
// rows; boxes of 64 columns x box_rows rows, 128-byte swizzle, zeros outside.
inline bool tensor_map_2d(const void* ptr, long long rows, long long cols, long long stride,
                          int box_rows, CUtensorMap* out)
{
    static std::mutex mutex;
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
    const MapKey key { ptr, rows, cols, stride, box_rows };
    std::lock_guard<std::mutex> lock(mutex);
    auto it = cache.find(key);
    if (it != cache.end()) {
        *out = it->second;
        return true;
    }
    EncodeTiledFn fn = encode_tiled();
    if (!fn)
        return false;
    const cuuint64_t dims[2] = { (cuuint64_t)cols, (cuuint64_t)rows };
    const cuuint64_t strides[1] = { (cuuint64_t)stride * 2 };
    const cuuint32_t box[2] = { (cuuint32_t)TENSOR_MAP_BOX_COLS, (cuuint32_t)box_rows };
    const cuuint32_t elem[2] = { 1, 1 };
    CUtensorMap map;
    const CUresult r = fn(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides,
                          box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return false;
    if (cache.size() > 8192)
        cache.clear();
    cache.emplace(key, map);
    *out = map;
    return true;
}

} // namespace chibi
