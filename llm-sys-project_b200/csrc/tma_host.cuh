// Host-side construction of TMA tensor maps.  The driver entry point is resolved at
// run time through the CUDA runtime, so the library does not link libcuda directly.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include "common.cuh"

typedef CUresult (*b200_encode_tiled_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                         const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                         CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                         CUtensorMapFloatOOBfill);

static inline b200_encode_tiled_fn b200_get_encode_tiled() {
    static b200_encode_tiled_fn fn = nullptr;
    if (fn) return fn;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
        return nullptr;
    fn = reinterpret_cast<b200_encode_tiled_fn>(p);
    return fn;
}

// Row-major byte matrix [rows, cols] (cols contiguous), tile = box_rows x 128 bytes,
// 128-byte swizzle: row r of a tile lands at r*128 with its 16-byte chunks XORed by (r & 7).
// Out-of-range rows read as zeros.  Requires base and cols to be multiples of 16.
static inline int b200_make_tmap_u8_sw128(CUtensorMap* map, const void* base, unsigned long long rows,
                                          unsigned long long cols, unsigned box_rows) {
    b200_encode_tiled_fn enc = b200_get_encode_tiled();
    if (!enc) return B200_CUDA_ERROR;
    if ((reinterpret_cast<uintptr_t>(base) & 15) || (cols & 15) || box_rows == 0 || box_rows > 256)
        return B200_BAD_ARG;
    cuuint64_t gdim[2] = {cols, rows};
    cuuint64_t gstride[1] = {cols};
    cuuint32_t box[2] = {128, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), gdim, gstride, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? B200_OK : B200_CUDA_ERROR;
}
