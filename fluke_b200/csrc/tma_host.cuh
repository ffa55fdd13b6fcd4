// tma_host.cuh -- host-side construction of TMA tensor maps without linking libcuda: the
// driver's cuTensorMapEncodeTiled is looked up through the runtime.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace fluke_sm100 {

typedef CUresult (*encode_tiled_fn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                    const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                    const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline encode_tiled_fn get_encode_tiled() {
    static encode_tiled_fn fn = nullptr;
    if (!fn) {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
                cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<encode_tiled_fn>(p);
    }
    return fn;
}

// Row-major 2-D tensor [rows, cols] with `row_stride_bytes` between rows (multiple of 16),
// copied in boxes of box_rows x box_cols elements; box_cols * elem_bytes must be 128 when the
// 128-byte swizzle is used. Out-of-range parts of a box read as zero and are not written.
// make_tmap_2d_sw takes the swizzle mode itself (the box row must span exactly that many bytes).
inline int make_tmap_2d_sw(CUtensorMap *m, CUtensorMapDataType dt, const void *base, uint64_t rows,
                           uint64_t cols, uint64_t row_stride_bytes, uint32_t box_rows,
                           uint32_t box_cols, CUtensorMapSwizzle swizzle) {
    encode_tiled_fn fn = get_encode_tiled();
    if (!fn) return (int)cudaErrorNotSupported;
    if ((reinterpret_cast<uintptr_t>(base) & 15u) || (row_stride_bytes & 15u))
        return (int)cudaErrorMisalignedAddress;
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {row_stride_bytes};
    cuuint32_t box[2] = {box_cols, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(m, dt, 2, const_cast<void *>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : (int)cudaErrorInvalidValue;
}

inline int make_tmap_2d(CUtensorMap *m, CUtensorMapDataType dt, uint32_t elem_bytes,
                        const void *base, uint64_t rows, uint64_t cols, uint64_t row_stride_bytes,
                        uint32_t box_rows, uint32_t box_cols, bool swizzle128) {
    (void)elem_bytes;
    return make_tmap_2d_sw(m, dt, base, rows, cols, row_stride_bytes, box_rows, box_cols,
                           swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE);
}

// Row-major 3-D tensor [planes, rows, cols]; boxes are 1 x box_rows x box_cols.
inline int make_tmap_3d_sw(CUtensorMap *m, CUtensorMapDataType dt, const void *base, uint64_t planes,
                           uint64_t rows, uint64_t cols, uint64_t row_stride_bytes,
                           uint64_t plane_stride_bytes, uint32_t box_rows, uint32_t box_cols,
                           CUtensorMapSwizzle swizzle) {
    encode_tiled_fn fn = get_encode_tiled();
    if (!fn) return (int)cudaErrorNotSupported;
    if ((reinterpret_cast<uintptr_t>(base) & 15u) || (row_stride_bytes & 15u) ||
        (plane_stride_bytes & 15u))
        return (int)cudaErrorMisalignedAddress;
    cuuint64_t dims[3] = {cols, rows, planes};
    cuuint64_t strides[2] = {row_stride_bytes, plane_stride_bytes};
    cuuint32_t box[3] = {box_cols, box_rows, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(m, dt, 3, const_cast<void *>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : (int)cudaErrorInvalidValue;
}

inline int make_tmap_3d(CUtensorMap *m, CUtensorMapDataType dt, const void *base, uint64_t planes,
                        uint64_t rows, uint64_t cols, uint64_t row_stride_bytes,
                        uint64_t plane_stride_bytes, uint32_t box_rows, uint32_t box_cols,
                        bool swizzle128) {
    return make_tmap_3d_sw(m, dt, base, planes, rows, cols, row_stride_bytes, plane_stride_bytes,
                           box_rows, box_cols,
                           swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE);
}

// General form: `rank` dimensions (2..5), innermost first. dims/box in elements, strides in bytes
// for dimensions 1..rank-1 (multiples of 16; they need not grow with the dimension, so a
// dimension may walk the K blocks of a row while an outer one walks the rows). The innermost box
// extent must span exactly 128 bytes under the 128-byte swizzle.
inline int make_tmap_nd(CUtensorMap *m, CUtensorMapDataType dt, const void *base, int rank,
                        const uint64_t *dims, const uint64_t *strides_bytes, const uint32_t *box,
                        CUtensorMapSwizzle swizzle) {
    encode_tiled_fn fn = get_encode_tiled();
    if (!fn) return (int)cudaErrorNotSupported;
    if (rank < 2 || rank > 5) return (int)cudaErrorInvalidValue;
    if (reinterpret_cast<uintptr_t>(base) & 15u) return (int)cudaErrorMisalignedAddress;
    cuuint64_t d[5], st[4];
    cuuint32_t b[5], estr[5];
    for (int i = 0; i < rank; ++i) { d[i] = dims[i]; b[i] = box[i]; estr[i] = 1; }
    for (int i = 0; i + 1 < rank; ++i) {
        if (strides_bytes[i] & 15u) return (int)cudaErrorMisalignedAddress;
        st[i] = strides_bytes[i];
    }
    CUresult r = fn(m, dt, (cuuint32_t)rank, const_cast<void *>(base), d, st, b, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : (int)cudaErrorInvalidValue;
}

}  // namespace fluke_sm100
