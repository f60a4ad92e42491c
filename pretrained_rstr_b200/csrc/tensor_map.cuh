// Tensor maps for TMA (cp.async.bulk.tensor): the driver's encoder, looked up once through
// the runtime, and a cached "K-slab" view of a row-major bfloat16 matrix.
#pragma once
#include <cuda.h>
#include <cudaTypedefs.h>
#include <cuda_runtime.h>

#include <mutex>
#include <unordered_map>

namespace tmap {

inline PFN_cuTensorMapEncodeTiled_v12000 encode_fn() {
    static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
                cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
    });
    return fn;
}

struct MapKey {
    const void* ptr;
    long rows, cols, pitch;
    int box_rows;
    bool operator==(const MapKey& o) const {
        return ptr == o.ptr && rows == o.rows && cols == o.cols && pitch == o.pitch &&
               box_rows == o.box_rows;
    }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        size_t h = (size_t)k.ptr;
        h = h * 1000003u ^ (size_t)k.rows;
        h = h * 1000003u ^ (size_t)k.cols;
        h = h * 1000003u ^ (size_t)k.pitch;
        h = h * 1000003u ^ (size_t)k.box_rows;
        return h;
    }
};

// Tensor map of a row-major bf16 matrix [rows, cols] with `pitch` elements between rows;
// box = 64 columns x box_rows rows, 128-byte swizzle, out-of-range elements read as zero.
inline int get_map(const void* ptr, long rows, long cols, long pitch, int box_rows, CUtensorMap* out) {
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
    static std::mutex mu;
    MapKey key{ptr, rows, cols, pitch, box_rows};
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it != cache.end()) {
        *out = it->second;
        return 0;
    }
    auto fn = encode_fn();
    if (!fn) return -6;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)pitch * 2};
    cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUtensorMap map;
    CUresult r = fn(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims,
                    strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return -5;
    if (cache.size() > 8192) cache.clear();
    cache.emplace(key, map);
    *out = map;
    return 0;
}

struct SlabKey {
    const void* ptr;
    long rows, cols, pitch;
    int box_rows, box_slabs;
    bool operator==(const SlabKey& o) const {
        return ptr == o.ptr && rows == o.rows && cols == o.cols && pitch == o.pitch &&
               box_rows == o.box_rows && box_slabs == o.box_slabs;
    }
};
struct SlabKeyHash {
    size_t operator()(const SlabKey& k) const {
        size_t h = (size_t)k.ptr;
        h = h * 1000003u ^ (size_t)k.rows;
        h = h * 1000003u ^ (size_t)k.cols;
        h = h * 1000003u ^ (size_t)k.pitch;
        h = h * 1000003u ^ (size_t)(k.box_rows * 1024 + k.box_slabs);
        return h;
    }
};

// A row-major bfloat16 matrix [rows, cols] (cols a multiple of 64, `pitch` elements
// between rows) seen as {64 columns, rows, cols / 64 slabs}: one copy brings box_rows rows
// of box_slabs consecutive 64-column slabs, each slab landing as [box_rows][64] with the
// 128-byte swizzle; rows and slabs out of range read as zero.  Returns 0, -6 without the
// driver's encoder, -5 when the driver refuses the map.
inline int slab_map(const void* ptr, long rows, long cols, long pitch, int box_rows,
                    int box_slabs, CUtensorMap* out) {
    static std::unordered_map<SlabKey, CUtensorMap, SlabKeyHash> cache;
    static std::mutex mu;
    SlabKey key{ptr, rows, cols, pitch, box_rows, box_slabs};
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it != cache.end()) {
        *out = it->second;
        return 0;
    }
    auto fn = encode_fn();
    if (!fn) return -6;
    cuuint64_t dims[3] = {64, (cuuint64_t)rows, (cuuint64_t)(cols / 64)};
    cuuint64_t strides[2] = {(cuuint64_t)pitch * 2, 128};
    cuuint32_t box[3] = {64, (cuuint32_t)box_rows, (cuuint32_t)box_slabs};
    cuuint32_t estr[3] = {1, 1, 1};
    CUtensorMap map;
    CUresult r = fn(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims,
                    strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return -5;
    if (cache.size() > 8192) cache.clear();
    cache.emplace(key, map);
    *out = map;
    return 0;
}
}  // namespace tmap
