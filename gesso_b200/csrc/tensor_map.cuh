// Host side of TMA: the driver's tensor-map encoder (fetched through the runtime, so that the library
// does not link against libcuda) and the one map the matrix products use.
#pragma once
#include <cuda.h>

#include "common.cuh"

typedef CUresult (*TensorMapEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                      const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                      CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static inline TensorMapEncodeFn tensor_map_encoder() {
    static TensorMapEncodeFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (TensorMapEncodeFn)p;
    }
    return fn;
}

// A row-major [rows, K] bfloat16 matrix in tiles of box_rows x 64 elements (128 bytes) with 128-byte swizzle;
// rows and columns beyond the matrix read as zero.
static inline int make_matrix_map(CUtensorMap* map, const void* base, int rows, int K, int box_rows) {
    TensorMapEncodeFn fn = tensor_map_encoder();
    if (!fn) return GESSO_ERR_UNSUPPORTED;
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)K * sizeof(bf16)};
    const cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : GESSO_ERR_UNSUPPORTED;
}
