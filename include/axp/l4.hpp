// L4 intent patterns: portable descriptions only (reference include/axp/l4.hpp:18-74,
// same parameter lists and defaults), plus the canonical presets.
// Public surface restated from tribe-iro/iro-cuda-ax (MIT licence, Copyright (c) 2026 IRO; the notice is kept in
// THIRD_PARTY_NOTICES.md at the repository root).
#pragma once
#include <iro_cuda_ax_core.hpp>

#include "intent.hpp"
#include "naming/subjects.hpp"
#include "recipes.hpp"
#include "level3/epilogue.hpp"

namespace axp::l4 {

namespace detail {
template <class... Subjects>
constexpr bool subjects_follow_policy() {
    return (axp::subject::is_subject<Subjects>::value && ...);
}
}  // namespace detail

template <class Recipe, int BlockM, int BlockN, int BlockK, int Stages, int KTiles, class ASubj = axp::subject::MatrixA,
          class BSubj = axp::subject::MatrixB, class CSubj = axp::subject::MatrixC,
          class WgmmaSubj = axp::subject::Accumulator, class MemoryPatternA = axp::intent::memory_pattern::Optimized,
          class MemoryPatternB = axp::intent::memory_pattern::Optimized,
          class LoadModeA = axp::intent::load_mode::AsyncPrefetch, class LoadModeB = axp::intent::load_mode::AsyncPrefetch,
          class Schedule = axp::intent::schedule::Pipelined, class ScaleASubj = iro::contract::subject::global,
          class ScaleBSubj = iro::contract::subject::global>
struct GemmPattern {
    static_assert(detail::subjects_follow_policy<ASubj, BSubj, CSubj, WgmmaSubj, ScaleASubj, ScaleBSubj>(),
                  "GemmPattern: subjects must follow canonical derivation policy");
};

// GEMM with a fused epilogue policy (reference include/axp/l4.hpp:36-53).
template <class Recipe, int BlockM, int BlockN, int BlockK, int Stages, int KTiles, class EpiloguePolicy,
          class ASubj = axp::subject::MatrixA, class BSubj = axp::subject::MatrixB, class CSubj = axp::subject::MatrixC,
          class WgmmaSubj = axp::subject::Accumulator, class MemoryPatternA = axp::intent::memory_pattern::Optimized,
          class MemoryPatternB = axp::intent::memory_pattern::Optimized,
          class LoadModeA = axp::intent::load_mode::AsyncPrefetch, class LoadModeB = axp::intent::load_mode::AsyncPrefetch,
          class Schedule = axp::intent::schedule::Pipelined, class ScaleASubj = iro::contract::subject::global,
          class ScaleBSubj = iro::contract::subject::global>
struct GemmFusedPattern {
    static_assert(detail::subjects_follow_policy<ASubj, BSubj, CSubj, WgmmaSubj, ScaleASubj, ScaleBSubj>(),
                  "GemmFusedPattern: subjects must follow canonical derivation policy");
};

template <class Recipe, int TileQ, int TileK, int TileV, int HeadDim, int Stages, int SlotIdx,
          class QSubj = axp::subject::AttentionQ, class KSubj = axp::subject::AttentionK,
          class VSubj = axp::subject::AttentionV, class AccSubj = axp::subject::Accumulator,
          class OldStateSubj = axp::subject::AttentionS, class OutStateSubj = axp::subject::wire<axp::tag::S, 1>,
          class MemoryPatternQ = axp::intent::memory_pattern::Optimized,
          class MemoryPatternK = axp::intent::memory_pattern::Optimized,
          class MemoryPatternV = axp::intent::memory_pattern::Optimized,
          class LoadModeQ = axp::intent::load_mode::AsyncPrefetch, class LoadModeK = axp::intent::load_mode::AsyncPrefetch,
          class LoadModeV = axp::intent::load_mode::AsyncPrefetch, class Schedule = axp::intent::schedule::Pipelined,
          class TileSkip = axp::intent::tile_skip::None>
struct AttentionPattern {
    static_assert(detail::subjects_follow_policy<QSubj, KSubj, VSubj, AccSubj, OldStateSubj, OutStateSubj>(),
                  "AttentionPattern: subjects must follow canonical derivation policy");
};

#include "l4/preset/common.hpp"
#include "l4/preset/gemm.hpp"
#include "l4/preset/attention.hpp"

// Manifest hooks (reference include/axp/l4.hpp:474-497): the generated registry
// index specialises these per manifest row.
namespace manifest {
template <class Pattern, class Cap>
struct enabled : std::false_type {};
template <class Pattern, class Cap>
inline constexpr bool enabled_v = enabled<Pattern, Cap>::value;
template <class Pattern>
struct tie_break_key {
    static constexpr iro::util::u64 value = 0;
};
template <class Pattern>
inline constexpr bool has_tie_break_key_v = tie_break_key<Pattern>::value != 0;
}  // namespace manifest

}  // namespace axp::l4
