// Host-side construction of the TMA descriptors shared by the tensor-core kernels: (outer, rows, K) tensors with K
// contiguous, read or written in boxes of 128 bytes x box_rows x 1 under the 128-byte swizzle (the layout the UMMA
// shared-memory descriptors of ptx_sm100.cuh expect). cuTensorMapEncodeTiled comes from the driver through the
// runtime's entry-point query, so the library does not link libcuda.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include "common.cuh"

namespace aristos {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            return nullptr;
        fn = reinterpret_cast<EncodeTiledFn>(sym);
    }
    return fn;
}

// elt_bytes: 1, 2 or 4. Rows past `rows` and columns past K read as zero and are not written.
inline aristos_status_t encode_map_3d(CUtensorMap* tm, CUtensorMapDataType dt, int elt_bytes, const void* base, int K,
                                      int rows, int outer, int box_rows) {
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) { set_last_error("cuTensorMapEncodeTiled is not available from the driver"); return ARISTOS_ERR_CUDA; }
    const cuuint64_t elt = (cuuint64_t)elt_bytes;
    const cuuint64_t dims[3] = {(cuuint64_t)K, (cuuint64_t)rows, (cuuint64_t)outer};
    const cuuint64_t strides[2] = {(cuuint64_t)K * elt, (cuuint64_t)K * elt * (cuuint64_t)rows};
    const cuuint32_t box[3] = {(cuuint32_t)(128 / elt), (cuuint32_t)box_rows, 1};
    const cuuint32_t estr[3] = {1, 1, 1};
    const CUresult r = enc(tm, dt, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_last_error("cuTensorMapEncodeTiled failed with %d (K=%d rows=%d outer=%d, %d-byte elements)", (int)r, K,
                       rows, outer, elt_bytes);
        return ARISTOS_ERR_CUDA;
    }
    return ARISTOS_OK;
}

}  // namespace aristos
