// Host-side construction of TMA tensor maps. The encoder lives in the driver library; it is
// looked up through the runtime so the shared library has no link-time dependence on libcuda.
#pragma once

#include "common.cuh"

#include <cuda.h>
#include <mutex>

namespace aeon_b200 {

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                   CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                   CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(sym);
    });
    if (!fn) throw StatusError(AEON_B200_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    return fn;
}

// Row-major 16-bit matrix [rows, cols] whose rows are `row_stride` elements apart (a multiple
// of 8, i.e. 16 bytes); box = 64 columns (128 B) x `box_rows` rows (a multiple of 8, at most 256:
// a box is whole 1024-byte swizzle atoms), 128-byte swizzle; rows past the end read as zero.
inline CUtensorMap make_rowmajor16_map(const void* base, uint64_t rows, uint64_t cols, uint64_t row_stride,
                                       uint32_t box_rows = 64) {
    CUtensorMap map;
    const cuuint64_t gdim[2] = {cols, rows};
    const cuuint64_t gstride[1] = {row_stride * 2};
    const cuuint32_t box[2] = {64, box_rows};
    const cuuint32_t estride[2] = {1, 1};
    const CUresult rc = encode_tiled()(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base), gdim,
                                       gstride, box, estride, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                       CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                                       CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS)
        throw StatusError(AEON_B200_ERR_CUDA, "cuTensorMapEncodeTiled failed with code " + std::to_string(rc));
    return map;
}

}  // namespace aeon_b200
