// Host-side leaf of the sm100 kit: tiled tensor-map encoding (HostMakeTensorMap,
// reference contract include/axp/protocol/tma/contracts.hpp:71-93, sm90 realization
// include/axp/realize/sm90.hpp:416-440 calling cuTensorMapEncodeTiled).  The driver
// function is taken through cudaGetDriverEntryPoint, so that nothing links against
// libcuda.  E4M3 / E5M2 tensors travel as CU_TENSOR_MAP_DATA_TYPE_UINT8 (the
// reference's dtype map has no 8-bit float case, sm90.hpp:54-78).
#pragma once

#include <cuda.h>
#include <cuda_runtime_api.h>

#include <cstdint>

namespace axp::realize::sm100 {

struct HostTensorMapEncoder {
    using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                       const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                       CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

    static EncodeTiledFn entry_point() {
        static EncodeTiledFn fn = [] {
            void* p = nullptr;
            cudaDriverEntryPointQueryResult q;
            if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
                p = nullptr;
            return reinterpret_cast<EncodeTiledFn>(p);
        }();
        return fn;
    }

    // Rank-`rank` tiled map (dims / box innermost first; strides in bytes for dims 1..rank-1), zero fill outside the
    // tensor, 256-byte L2 promotion.  Returns the CUresult as an int, or -1 when the driver entry point is missing.
    static int execute(CUtensorMap* out, CUtensorMapDataType dtype, int rank, const void* base, const uint64_t* dims,
                       const uint64_t* strides_bytes, const uint32_t* box, CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B) {
        EncodeTiledFn fn = entry_point();
        if (!fn) return -1;
        cuuint64_t d[5], s[5];
        cuuint32_t b[5], es[5];
        for (int i = 0; i < rank; ++i) {
            d[i] = dims[i];
            b[i] = box[i];
            es[i] = 1;
        }
        for (int i = 0; i + 1 < rank; ++i) s[i] = strides_bytes[i];
        return int(fn(out, dtype, cuuint32_t(rank), const_cast<void*>(base), d, s, b, es, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                      CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE));
    }
};

}  // namespace axp::realize::sm100
