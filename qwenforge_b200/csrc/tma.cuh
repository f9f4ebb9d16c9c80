// Tensor maps and tiled copies of the tensor memory accelerator (TMA), shared by the kernels that use them.
// No copy here uses cluster multicast: every block fetches its own tiles.
#pragma once
#include <cuda.h>

#include "mma.cuh"

// 2-D tiled copy global -> shared of the box at element coordinates (x, y) = (column, row); completes on `bar`.
// x * element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
                     smem_addr(dst)),
                 "l"(map), "r"(smem_addr(bar)), "r"(x), "r"(y)
                 : "memory");
}

typedef CUresult (*QfEncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                    const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver's tensor-map encoder, looked up through the runtime (no link against the driver library).
static inline QfEncodeTiledFn qf_encode_tiled() {
    static QfEncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult status;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &status) == cudaSuccess &&
            status == cudaDriverEntryPointSuccess)
            fn = (QfEncodeTiledFn)p;
    }
    return fn;
}

// A 2-D map over a row-major bf16 matrix [rows][ld] of `cols` used columns: boxes of `box_rows` rows x 64 columns
// (128 bytes, stored with the 128-byte swizzle), zeros outside the matrix.
static inline bool qf_make_map_bf16(CUtensorMap* map, const void* base, long long rows, long long cols, long long ld,
                                    int box_rows) {
    QfEncodeTiledFn fn = qf_encode_tiled();
    if (!fn) return false;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
