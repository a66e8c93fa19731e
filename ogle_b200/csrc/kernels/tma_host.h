// Host-side TMA descriptor helpers shared by the kernels that use tensor maps.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

namespace ogle {

// Address of the library's device status word on the current device.
int* error_flag_ptr();

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

// swizzle: CU_TENSOR_MAP_SWIZZLE_128B for UMMA operand tiles, _NONE for plain tiles.
inline bool make_map_sw(CUtensorMapSwizzle swizzle, CUtensorMap* m, const void* ptr, int rank, const cuuint64_t* dims, const cuuint64_t* strides_bytes,
              const cuuint32_t* box, const cuuint32_t* estr) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, (cuuint32_t)rank, const_cast<void*>(ptr), dims, strides_bytes,
                    box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}


inline bool make_map(CUtensorMap* m, const void* ptr, int rank, const cuuint64_t* dims, const cuuint64_t* strides_bytes,
                     const cuuint32_t* box, const cuuint32_t* estr) {
    return make_map_sw(CU_TENSOR_MAP_SWIZZLE_128B, m, ptr, rank, dims, strides_bytes, box, estr);
}

}  // namespace ogle
