// Attention presets for the sm100 rows (additive to the reference's f16 presets in
// include/axp/l4/preset/attention.hpp:7-69).  Included inside namespace axp::l4.
#pragma once

namespace preset {

// bf16 flash-attention forward tile: 128 queries x 128 keys, head dim 128, causal skip; four K/V stages (of the
// 64-key steps the realization takes a tile in).
using Attention128x128x128CausalBf16 = axp::l4::AttentionPattern<
    axp::recipe::BF16AccF32Fast,
    128, 128, 128, 128,
    4, 0,
    AttnQ, AttnK, AttnV,
    AttnAcc, AttnStateOld, AttnStateNew,
    axp::intent::memory_pattern::Optimized,
    axp::intent::memory_pattern::Optimized,
    axp::intent::memory_pattern::Optimized,
    axp::intent::load_mode::AsyncPrefetch,
    axp::intent::load_mode::AsyncPrefetch,
    axp::intent::load_mode::AsyncPrefetch,
    axp::intent::schedule::ProducerConsumer,
    axp::intent::tile_skip::Causal
>;

// FP8 (E4M3) flash-attention forward tile with GQA head mapping and per-head descales.
using Attention128x128x128CausalFp8Gqa = axp::l4::AttentionPattern<
    axp::recipe::E4M3AccF32OutBF16,
    128, 128, 128, 128,
    3, 0,
    AttnQ, AttnK, AttnV,
    AttnAcc, AttnStateOld, AttnStateNew,
    axp::intent::memory_pattern::Optimized,
    axp::intent::memory_pattern::Optimized,
    axp::intent::memory_pattern::Optimized,
    axp::intent::load_mode::AsyncPrefetch,
    axp::intent::load_mode::AsyncPrefetch,
    axp::intent::load_mode::AsyncPrefetch,
    axp::intent::schedule::ProducerConsumer,
    axp::intent::tile_skip::Causal
>;

}  // namespace preset
