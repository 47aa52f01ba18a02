// TMA tensor maps for row-major bfloat16 matrices, made once and kept.
//
// cuTensorMapEncodeTiled is a host call of a microsecond or two, and a step makes the same maps
// over and over (weights never move, activations live in buffers that keep their addresses), so
// the maps are looked up in a small table by what defines them.  The table is per library and is
// guarded by a mutex; when it is full the oldest entry goes.

#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <mutex>

namespace tensor_maps {

typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiled encode_fn() {
    static EncodeTiled fn = nullptr;
    if (fn == nullptr) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
                cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiled>(p);
    }
    return fn;
}

struct Key {
    const void* base;
    long long rows;
    int cols, ld, box_rows, box_cols;
    bool operator==(const Key& o) const {
        return base == o.base && rows == o.rows && cols == o.cols && ld == o.ld &&
               box_rows == o.box_rows && box_cols == o.box_cols;
    }
};

// A [rows, cols] bfloat16 matrix with row stride ld (elements), boxes of box_rows x box_cols,
// 128-byte swizzle, zero fill outside.  0 or a negative code (-20: no driver entry point, -21:
// the driver refused the map).
inline int get(CUtensorMap* map, const void* base, long long rows, int cols, int ld, int box_rows,
               int box_cols) {
    constexpr int SLOTS = 256;
    static Key keys[SLOTS];
    static CUtensorMap maps[SLOTS];
    static int used = 0, next = 0;
    static std::mutex guard;
    const Key key = {base, rows, cols, ld, box_rows, box_cols};
    std::lock_guard<std::mutex> lock(guard);
    for (int i = 0; i < used; ++i)
        if (keys[i] == key) {
            *map = maps[i];
            return 0;
        }
    EncodeTiled encode = encode_fn();
    if (encode == nullptr) return -20;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    const CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base),
                              dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return -21;
    const int slot = used < SLOTS ? used++ : (next++ % SLOTS);
    keys[slot] = key;
    maps[slot] = *map;
    return 0;
}

}  // namespace tensor_maps
