// Launch configuration of the kernels the default dispatch starts, in one place: the kernel translation units
// static_assert their own constants against these, axp_sm100_query answers from them, and the compile-time check of
// the manifest rows (tests/compile/sm100_rows.cu) compares the level-3 graphs with them, so that the three
// descriptions of a kernel cannot drift apart without a build failure.
#pragma once

namespace axp_shim::cfg {

struct Gemm {
    int tile_m, tile_n, tile_k;      // per CTA: accumulator rows, columns, K elements per shared-memory stage
    int cta_group;                   // CTAs per MMA
    int stages, stage_bytes;         // shared-memory ring per CTA
    int dyn_smem;                    // dynamic shared memory per CTA (ring + 1 KiB alignment slack)
    int tmem_cols;
    int threads;
    int producer_regs, epilogue_regs;   // setmaxnreg budgets of warpgroup 0 / the epilogue warpgroups
};
// FP8 E4M3 block-scaled: CTA pair, 256 x 256 per pair, two epilogue warpgroups
constexpr Gemm kGemmFp8 = {128, 256, 128, 2, 6, 32768, 6 * 32768 + 1024, 512, 384, 40, 232};
// bf16: CTA pair, four epilogue warpgroups
constexpr Gemm kGemmBf16 = {128, 256, 64, 2, 6, 32768, 6 * 32768 + 1024, 512, 640, 32, 112};

struct Attn {
    int tile_q, kv_tile, head_dim;   // query rows per Q tile, keys per KV step, head dimension
    int q_tiles;                     // Q tiles per CTA
    int kv_stages;
    int dyn_smem;
    int tmem_cols;
    int threads;
    int producer_regs, softmax_regs;
    int issuers;                     // MMA-issuing warps
    bool p_through_smem;             // P reaches the P.V MMA through shared memory (else it overwrites S in tensor memory)
};
constexpr Attn kAttnBf16 = {128, 64, 128, 2, 4, 197632, 512, 384, 56, 224, 2, false};
constexpr Attn kAttnFp8 = {128, 128, 128, 2, 3, 197632, 512, 384, 56, 224, 2, true};

}  // namespace axp_shim::cfg
