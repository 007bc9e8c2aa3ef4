// Host side of TMA: tensor maps of row-major bf16 matrices, fetched in boxes with the 128-byte swizzle.  The driver's
// encoder is looked up through the runtime (no link against libcuda); maps are kept per (address, shape, box).
#pragma once
#include "common.cuh"

#include <cuda.h>
#include <mutex>
#include <unordered_map>

namespace cvb {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    });
    return fn;
}

// Encodes the map of a bf16 matrix [rows, cols] (row-major, rows of `cols` elements) fetched in boxes of
// [box_rows, box_cols]; box_cols * 2 bytes must be 128 (the swizzle span).  Nothing is kept: no table, no heap.
inline int encode_bf16_map(CUtensorMap* out, const void* base, int64_t rows, int64_t cols, int box_cols, int box_rows) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (fn == nullptr) return CVB_E_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (cols * sizeof(__nv_bfloat16)) % 16 != 0) return CVB_E_ALIGN;
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(cols) * sizeof(__nv_bfloat16)};
    const cuuint32_t box[2] = {static_cast<cuuint32_t>(box_cols), static_cast<cuuint32_t>(box_rows)};
    const cuuint32_t estr[2] = {1u, 1u};
    if (fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return CVB_E_SHAPE;
    return CVB_OK;
}

// The same, kept per (address, shape, box): a step asks for the same few maps again and again.
inline int cached_bf16_map(CUtensorMap* out, const void* base, int64_t rows, int64_t cols, int box_cols, int box_rows) {
    struct Key {
        const void* p; int64_t r, c; int bc, br;
        bool operator==(const Key& o) const { return p == o.p && r == o.r && c == o.c && bc == o.bc && br == o.br; }
    };
    struct Hash {
        size_t operator()(const Key& k) const {
            return std::hash<const void*>()(k.p) ^ (std::hash<int64_t>()(k.r) * 1315423911u) ^ (std::hash<int64_t>()(k.c) * 2654435761u) ^
                   (static_cast<size_t>(k.bc) * 131) ^ (static_cast<size_t>(k.br) * 7);
        }
    };
    static std::unordered_map<Key, CUtensorMap, Hash> maps;
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    const Key key{base, rows, cols, box_cols, box_rows};
    auto it = maps.find(key);
    if (it == maps.end()) {
        CUtensorMap m;
        const int rc = encode_bf16_map(&m, base, rows, cols, box_cols, box_rows);
        if (rc != CVB_OK) return rc;
        if (maps.size() > 4096) maps.clear();          // activations of many different lengths: start over
        it = maps.emplace(key, m).first;
    }
    *out = it->second;
    return CVB_OK;
}

}  // namespace cvb
