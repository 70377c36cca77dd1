// GEMM presets for the sm100 rows (additive to the reference's f16 presets in
// include/axp/l4/preset/gemm.hpp:7-45).  KTiles is the steady-state window the
// graph describes, not the problem's K extent.  Included inside namespace axp::l4.
#pragma once

namespace preset {

// FP8 E4M3 block-scaled GEMM, CTA tile 128 x 256 (CTA pairs: 256 x 256 per cluster), 128-wide K blocks, bf16 out.
using GemmFp8BlockScaled128x256x128 = axp::l4::GemmPattern<
    axp::recipe::E4M3BlockScaledAccF32OutBF16,
    128, 256, 128,
    6, 7,
    GemmA, GemmB, GemmC,
    GemmAcc,
    axp::intent::memory_pattern::Optimized,
    axp::intent::memory_pattern::Optimized,
    axp::intent::load_mode::AsyncPrefetch,
    axp::intent::load_mode::AsyncPrefetch,
    axp::intent::schedule::ProducerConsumer,
    GemmScaleA, GemmScaleB
>;

// BF16 GEMM, CTA tile 128 x 256 (CTA pairs: 256 x 256 per cluster), 64-wide K stages.
using GemmBf16_128x256x64 = axp::l4::GemmPattern<
    axp::recipe::BF16AccF32Fast,
    128, 256, 64,
    6, 7,
    GemmA, GemmB, GemmC,
    GemmAcc,
    axp::intent::memory_pattern::Optimized,
    axp::intent::memory_pattern::Optimized,
    axp::intent::load_mode::AsyncPrefetch,
    axp::intent::load_mode::AsyncPrefetch,
    axp::intent::schedule::ProducerConsumer
>;

// BF16 GEMM with the fused bias + SiLU epilogue (the sm100 counterpart of the reference's
// Gemm64x64x16BiasSiLU, include/axp/l4/preset/gemm.hpp:33-45).
using GemmBf16_128x256x64BiasSiLU = axp::l4::GemmFusedPattern<
    axp::recipe::BF16AccF32Fast,
    128, 256, 64,
    6, 7,
    axp::level3::epilogue::BiasActivationVec<GemmBiasSiLUTag, axp::level3::epilogue::act::SiLU>,
    GemmA, GemmB, GemmC,
    GemmAcc,
    axp::intent::memory_pattern::Optimized,
    axp::intent::memory_pattern::Optimized,
    axp::intent::load_mode::AsyncPrefetch,
    axp::intent::load_mode::AsyncPrefetch,
    axp::intent::schedule::ProducerConsumer
>;

// Gate / up projection of a gated MLP in one pass: out = SiLU(X.Wg^T) * (X.Wu^T), 128 output columns per tile
// (128 gate + 128 up accumulator columns).
using GemmBf16_128x256x64SwiGLU = axp::l4::GemmFusedPattern<
    axp::recipe::BF16AccF32Fast,
    128, 256, 64,
    6, 7,
    axp::level3::epilogue::GatedActivationVec<GemmUpOperandTag, axp::level3::epilogue::act::SiLU>,
    GemmA, GemmB, GemmC,
    GemmAcc,
    axp::intent::memory_pattern::Optimized,
    axp::intent::memory_pattern::Optimized,
    axp::intent::load_mode::AsyncPrefetch,
    axp::intent::load_mode::AsyncPrefetch,
    axp::intent::schedule::ProducerConsumer
>;

// D = alpha * (A.B^T) + beta * C (residual / accumulate-into-C forms).
using GemmBf16_128x256x64LinComb = axp::l4::GemmFusedPattern<
    axp::recipe::BF16AccF32Fast,
    128, 256, 64,
    6, 7,
    axp::level3::epilogue::LinearCombinationVec<GemmLinCombCTag, GemmLinCombAlphaTag, GemmLinCombBetaTag>,
    GemmA, GemmB, GemmC,
    GemmAcc,
    axp::intent::memory_pattern::Optimized,
    axp::intent::memory_pattern::Optimized,
    axp::intent::load_mode::AsyncPrefetch,
    axp::intent::load_mode::AsyncPrefetch,
    axp::intent::schedule::ProducerConsumer
>;

}  // namespace preset
