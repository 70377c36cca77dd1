// Entry points of the C-ABI that are not kernels of their own family: realization
// key lookup, error text, the causal-mask index kernel and the bounded-wait
// self-test.
#include <cstring>

#include "axp/realize/sm100.hpp"
#include "axp/realize/sm100_mask.hpp"
#include "host_common.hpp"
#include "kernel_config.hpp"

namespace rz = axp::realize::sm100;

namespace {

namespace cfg = axp_shim::cfg;

struct Row {
    const char* key;
    axp_sm100_caps caps;
};

constexpr axp_sm100_caps gemm_caps(int family, int elem_bits, const cfg::Gemm& g) {
    return {0, family, elem_bits, g.tile_m, g.tile_n, g.tile_k, g.cta_group, g.stages, g.dyn_smem, g.tmem_cols, g.threads};
}
constexpr axp_sm100_caps attn_caps(int elem_bits, const cfg::Attn& a) {
    // tile_n is the number of keys a step of the kernel takes (the KV tile of the shared-memory ring)
    return {0, 2, elem_bits, a.tile_q, a.kv_tile, a.head_dim, 1, a.kv_stages, a.dyn_smem, a.tmem_cols, a.threads};
}

// One entry per row of manifests/kernels_sm100.json (same realization_key strings), filled from the configuration
// the kernel translation units are checked against.
const Row kRows[] = {
    {"preset.gemm.fp8bs.128x256x128", gemm_caps(1, 8, cfg::kGemmFp8)},
    {"preset.gemm.bf16.128x256x64", gemm_caps(1, 16, cfg::kGemmBf16)},
    {"preset.gemm_fused.bf16.128x256x64.bias_silu", gemm_caps(3, 16, cfg::kGemmBf16)},
    {"preset.gemm_fused.bf16.128x256x64.lincomb", gemm_caps(3, 16, cfg::kGemmBf16)},
    {"preset.gemm_fused.bf16.128x256x64.swiglu", gemm_caps(3, 16, cfg::kGemmBf16)},
    {"preset.attention.bf16.128x128x128.causal", attn_caps(16, cfg::kAttnBf16)},
    {"preset.attention.fp8.gqa.128x128x128.causal", attn_caps(8, cfg::kAttnFp8)},
};

__global__ void causal_mask_tile_kernel(long long q_base, long long k_base, int tile_m, int tile_n,
                                        unsigned long long* mask, int* skip) {
    const int nbits = tile_m * tile_n;
    const int words = (nbits + 63) / 64;
    for (int w = blockIdx.x * blockDim.x + threadIdx.x; w < words; w += gridDim.x * blockDim.x) {
        unsigned long long bits = 0ull;
        for (int b = 0; b < 64; ++b) {
            const int idx = w * 64 + b;
            if (idx < nbits) {
                const int r = idx / tile_n, c = idx - r * tile_n;
                if (rz::causal_valid(q_base + r, k_base + c)) bits |= (1ull << b);
            }
        }
        mask[w] = bits;
    }
    if (blockIdx.x == 0 && threadIdx.x == 0) *skip = rz::causal_tile_skip(q_base, k_base, tile_m) ? 1 : 0;
}

__global__ void bounded_wait_selftest_kernel(long long limit_cycles, uint32_t* status) {
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        rz::BarrierInit::execute(&bar, 1);
        rz::BarrierInitFence::execute();
        // nothing ever arrives on `bar`: poll with the short limit, then report
        const long long t0 = clock64();
        bool done = false;
        while (!done && clock64() - t0 <= limit_cycles) done = rz::BarrierTryWait::execute(&bar, 0);
        if (!done && status) atomicOr(status, rz::kStatusError | rz::kRoleProducer | rz::kBarOther);
    }
}

}  // namespace

std::atomic<int>& axp_shim::option_slot(int id) {
    static std::atomic<int> slots[axp_shim::kOptCount];
    return slots[id];
}

std::atomic<long long>& axp_shim::debug_pointer() {
    static std::atomic<long long> ptr{0};
    return ptr;
}

extern "C" int axp_sm100_set_option(const char* name, int64_t value) {
    if (!name) return axp_shim::fail(AXP_ERR_BAD_ARG, "set_option: name is null");
    if (!strcmp(name, "debug_buffer") || !strcmp(name, "gemm.experiment")) {
#if defined(AXP_SM100_LATENCY_PROBES)
        // "debug_buffer": device pointer to 512 uint64 timestamps, or 0; "gemm.experiment": parts of the kernels switched off
        // (results are not valid when non-zero)
        if (!strcmp(name, "debug_buffer")) axp_shim::debug_pointer().store((long long)value);
        else axp_shim::option_slot(axp_shim::kOptGemmExperiment).store(int(value));
        return AXP_OK;
#else
        return axp_shim::fail(AXP_ERR_UNSUPPORTED, "set_option: '%s' exists only in builds with -DAXP_SM100_LATENCY_PROBES", name);
#endif
    }
    if (!strcmp(name, "gemm.epilogue_warpgroups")) {
        if (value != 0 && value != 2 && value != 4) return axp_shim::fail(AXP_ERR_BAD_ARG, "gemm.epilogue_warpgroups must be 0, 2 or 4");
        axp_shim::option_slot(axp_shim::kOptGemmEpiWg).store(int(value));
        return AXP_OK;
    }
    if (!strcmp(name, "gemm.cta_group")) {
        if (value != 0 && value != 1 && value != 2) return axp_shim::fail(AXP_ERR_BAD_ARG, "gemm.cta_group must be 0, 1 or 2");
        axp_shim::option_slot(axp_shim::kOptGemmCtaGroup).store(int(value));
        return AXP_OK;
    }
    if (!strcmp(name, "gemm.fp8_tile")) {   // FP8 block-scaled GEMM: 0 default, 128 (128 x 128 tiles, two CTAs per SM) or 256
        if (value != 0 && value != 128 && value != 256) return axp_shim::fail(AXP_ERR_BAD_ARG, "gemm.fp8_tile must be 0, 128 or 256");
        axp_shim::option_slot(axp_shim::kOptGemmFp8Tile).store(int(value));
        return AXP_OK;
    }
    if (!strcmp(name, "attn.exp_mode")) {
        if (value < 0 || value > 4) return axp_shim::fail(AXP_ERR_BAD_ARG, "attn.exp_mode must be in [0,4]");
        axp_shim::option_slot(axp_shim::kOptAttnPolyExp).store(int(value));
        return AXP_OK;
    }
    if (!strcmp(name, "attn.p_operand")) {   // 0 default, 1 = P in tensor memory, 2 = P through shared memory (E4M3 kernels)
        if (value < 0 || value > 2) return axp_shim::fail(AXP_ERR_BAD_ARG, "attn.p_operand must be 0, 1 or 2");
        axp_shim::option_slot(axp_shim::kOptAttnPOperand).store(int(value));
        return AXP_OK;
    }
    if (!strcmp(name, "attn.issuers")) {   // MMA-issuing threads of the attention kernels: 0 default, 1 or 2 (one per Q tile)
        if (value < 0 || value > 2) return axp_shim::fail(AXP_ERR_BAD_ARG, "attn.issuers must be 0, 1 or 2");
        axp_shim::option_slot(axp_shim::kOptAttnIssuers).store(int(value));
        return AXP_OK;
    }
    if (!strcmp(name, "attn.decode_kernel")) {   // bf16 split-KV with at most 16 query rows per KV head: 0 default, 1 = forward kernel, 2 = decode kernel
        if (value < 0 || value > 2) return axp_shim::fail(AXP_ERR_BAD_ARG, "attn.decode_kernel must be 0, 1 or 2");
        axp_shim::option_slot(axp_shim::kOptAttnDecode).store(int(value));
        return AXP_OK;
    }
    if (!strcmp(name, "attn.rescale")) {   // prefill attention: 0 default, 1 = reference maximum advanced on every new maximum, 2 = lazily (2^8)
        if (value < 0 || value > 2) return axp_shim::fail(AXP_ERR_BAD_ARG, "attn.rescale must be 0, 1 or 2");
        axp_shim::option_slot(axp_shim::kOptAttnRescale).store(int(value));
        return AXP_OK;
    }
    if (!strcmp(name, "attn.kv_tile")) {   // bf16 attention: keys per KV tile, 0 default, 64 or 128
        if (value != 0 && value != 64 && value != 128) return axp_shim::fail(AXP_ERR_BAD_ARG, "attn.kv_tile must be 0, 64 or 128");
        axp_shim::option_slot(axp_shim::kOptAttnKvTile).store(int(value));
        return AXP_OK;
    }
    return axp_shim::fail(AXP_ERR_UNSUPPORTED, "set_option: unknown option '%s'", name);
}

extern "C" uint64_t axp_sm100_fnv1a64(const char* s) {
    uint64_t h = 14695981039346656037ULL;
    for (; s && *s; ++s) {
        h ^= static_cast<unsigned char>(*s);
        h *= 1099511628211ULL;
    }
    return h;
}

extern "C" int axp_sm100_query(uint64_t realization_key, axp_sm100_caps* out) {
    if (!out) return axp_shim::fail(AXP_ERR_BAD_ARG, "query: out is null");
    for (const Row& r : kRows) {
        if (axp_sm100_fnv1a64(r.key) == realization_key) {
            *out = r.caps;
            out->realization_key = realization_key;
            return AXP_OK;
        }
    }
    return axp_shim::fail(AXP_ERR_UNSUPPORTED, "query: no sm100 row for realization key 0x%016llx",
                          (unsigned long long)realization_key);
}

extern "C" const char* axp_sm100_last_error(void) { return axp_shim::error_buffer(); }

extern "C" int axp_sm100_causal_mask_tile(int64_t q_base, int64_t k_base, int32_t tile_m, int32_t tile_n,
                                          uint64_t* mask_dev, int32_t* skip_dev, void* stream) {
    if (!mask_dev || !skip_dev) return axp_shim::fail(AXP_ERR_BAD_ARG, "causal_mask_tile: null output");
    if (tile_m <= 0 || tile_n <= 0 || tile_m > 1024 || tile_n > 1024)
        return axp_shim::fail(AXP_ERR_BAD_ARG, "causal_mask_tile: tile extents must be in [1,1024]");
    causal_mask_tile_kernel<<<8, 128, 0, static_cast<cudaStream_t>(stream)>>>(
        q_base, k_base, tile_m, tile_n, reinterpret_cast<unsigned long long*>(mask_dev), skip_dev);
    AXP_CUDA_TRY(cudaGetLastError());
    return AXP_OK;
}

extern "C" int axp_sm100_selftest_bounded_wait(int64_t limit_cycles, void* stream, uint32_t* status_dev) {
    if (limit_cycles <= 0 || limit_cycles > 4000000000LL)
        return axp_shim::fail(AXP_ERR_BAD_ARG, "selftest: limit_cycles must be in (0, 4e9]");
    bounded_wait_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(limit_cycles, status_dev);
    AXP_CUDA_TRY(cudaGetLastError());
    return AXP_OK;
}
