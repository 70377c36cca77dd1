// Host-side helpers shared by the launch shim translation units: error text,
// tensor-map encoding through the driver entry point (no link-time dependency on
// libcuda), cached device properties.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include <nvtx3/nvToolsExt.h>

#include "axp/realize/sm100_host.hpp"
#include "axp_sm100.h"

namespace axp_shim {

inline char* error_buffer() {
    static thread_local char buf[512] = "";
    return buf;
}

inline int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(error_buffer(), 512, fmt, ap);
    va_end(ap);
    return code;
}

#define AXP_CUDA_TRY(expr)                                                                         \
    do {                                                                                           \
        cudaError_t _e = (expr);                                                                   \
        if (_e != cudaSuccess)                                                                     \
            return ::axp_shim::fail(AXP_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(_e)); \
    } while (0)

// Tiled tensor map of rank `rank` (dims/strides innermost first; strides in
// bytes for dims 1..rank-1), 128-byte swizzle, zero fill outside the tensor: the
// kit's HostMakeTensorMap leaf with the shim's error convention.
inline int make_tensor_map(CUtensorMap* out, CUtensorMapDataType dtype, int rank, const void* base,
                           const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box,
                           CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B) {
    const int r = axp::realize::sm100::HostTensorMapEncoder::execute(out, dtype, rank, base, dims, strides_bytes, box, swizzle);
    if (r == -1) return fail(AXP_ERR_CUDA, "cuTensorMapEncodeTiled entry point not available");
    if (r != 0) return fail(AXP_ERR_CUDA, "cuTensorMapEncodeTiled returned %d", r);
    return AXP_OK;
}

struct DeviceInfo {
    int device = -1;
    int sm_count = 0;
    int cc_major = 0;
    int cc_minor = 0;
};

inline int current_device_info(DeviceInfo* info) {
    static thread_local DeviceInfo cached;
    int dev = 0;
    AXP_CUDA_TRY(cudaGetDevice(&dev));
    if (cached.device != dev) {
        DeviceInfo d;
        d.device = dev;
        AXP_CUDA_TRY(cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev));
        AXP_CUDA_TRY(cudaDeviceGetAttribute(&d.cc_major, cudaDevAttrComputeCapabilityMajor, dev));
        AXP_CUDA_TRY(cudaDeviceGetAttribute(&d.cc_minor, cudaDevAttrComputeCapabilityMinor, dev));
        cached = d;
    }
    *info = cached;
    if (info->cc_major != 10)
        return fail(AXP_ERR_UNSUPPORTED, "device compute capability %d.%d is not sm_100", info->cc_major,
                    info->cc_minor);
    return AXP_OK;
}

// A kernel that moves registers between its warpgroups (setmaxnreg) must have been
// compiled with at least `needed_regs_total` registers in its launch allocation
// (threads x registers per thread); otherwise an increase would wait forever.
template <class Kernel>
inline int check_register_pool(Kernel kernel, int threads, int needed_regs_total, const char* what) {
    cudaFuncAttributes fa;
    AXP_CUDA_TRY(cudaFuncGetAttributes(&fa, kernel));
    if (fa.numRegs * threads < needed_regs_total)
        return fail(AXP_ERR_UNSUPPORTED, "%s: built with %d registers x %d threads, the role budgets need %d", what,
                    fa.numRegs, threads, needed_regs_total);
    return AXP_OK;
}

// Process-wide tuning options set through axp_sm100_set_option (0 = library default).
enum OptionId { kOptGemmEpiWg = 0, kOptGemmCtaGroup = 1, kOptAttnPolyExp = 2, kOptGemmExperiment = 3, kOptAttnPOperand = 4, kOptAttnKvTile = 5, kOptAttnIssuers = 6, kOptGemmFp8Tile = 7, kOptAttnDecode = 8, kOptAttnRescale = 9, kOptCount = 10 };
std::atomic<int>& option_slot(int id);   // defined in shim.cu
std::atomic<long long>& debug_pointer();  // defined in shim.cu; device buffer for latency experiments

// NVTX range around the host side of an entry point (argument checks, tensor-map encoding, launch), so that a timeline
// tool shows which C-ABI call a kernel belongs to.  NVTX is header-only and costs a few nanoseconds when no tool is attached.
struct NvtxRange {
    explicit NvtxRange(const char* name) { nvtxRangePushA(name); }
    ~NvtxRange() { nvtxRangePop(); }
    NvtxRange(const NvtxRange&) = delete;
    NvtxRange& operator=(const NvtxRange&) = delete;
};

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace axp_shim
