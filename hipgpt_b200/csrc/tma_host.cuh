// Host side of the TMA copies: tensor maps over one fp32 plane of the launcher's layout.
#pragma once

#include "attn_common.cuh"

#include <cuda.h>

#include <mutex>

namespace hipgpt {

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// cuTensorMapEncodeTiled through the runtime (the library does not link against libcuda); nullptr when the driver has none.
inline EncodeTiledFn tma_encode_fn()
{
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

// Rank-3 map {E, S, B} over one [B*S][E] fp32 plane; a box is [1][box_rows][32 floats] = rows of 128 bytes, swizzled as
// asked (CU_TENSOR_MAP_SWIZZLE_128B, or .._128B_ATOM_32B for a 32-bit operand that is contiguous along N); rows past S
// read as zeros.  The plane must start on a 16-byte boundary and E must be a multiple of 4.
inline int tma_plane_map(CUtensorMap *m, const float *plane, int B, int S, int E, int box_rows, CUtensorMapSwizzle swizzle)
{
    EncodeTiledFn enc = tma_encode_fn();
    if (!enc) return fail(HIPGPT_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    const cuuint64_t dims[3] = {(cuuint64_t)E, (cuuint64_t)S, (cuuint64_t)B};
    const cuuint64_t strides[2] = {(cuuint64_t)E * 4, (cuuint64_t)S * E * 4};
    const cuuint32_t box[3] = {32, (cuuint32_t)box_rows, 1};
    const cuuint32_t estr[3] = {1, 1, 1};
    const CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float *>(plane), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(HIPGPT_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
    return HIPGPT_OK;
}

}  // namespace hipgpt
