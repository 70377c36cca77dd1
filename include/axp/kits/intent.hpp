// Intent selectors: how the portable wishes of an L4 pattern (memory pattern, load
// mode, schedule) become mechanisms on a capability.  Names and rules follow the
// reference (include/axp/kits/intent.hpp:47-104 select_swizzle / select_tma,
// :108-125 expert overrides, :152-190 select_schedule and the *_t aliases):
//   * memory_pattern::Optimized on a TMA target picks the widest swizzle span the
//     row of TileK elements fills: >= 128 bytes -> B128, >= 64 -> B64, >= 32 -> B32,
//     else none; every other memory pattern, and targets without TMA, get none;
//   * load_mode::AsyncPrefetch on a TMA target yields a TMA configuration for the
//     subject (here: TmaTiled<GlobalTile, Subj, PipeTag>), void without TMA;
//     Streaming and DeterministicLatency yield streaming_tag; anything else void;
//   * schedule::ProducerConsumer needs an asynchronous MMA unit that a producer
//     role can run ahead of (the reference asserts has_wgmma; sm100's is tcgen05);
//     other schedules pass through;
//   * axp::kit::expert::*_override specialisations win over the defaults.
#pragma once
#include <iro_cuda_ax_core.hpp>

#include "../intent.hpp"
#include "../swizzle.hpp"

namespace axp::kit::detail {

struct streaming_tag {};

// What select_tma hands to a staging recipe on a TMA target: the subject whose
// tensor map is encoded on the host (HostMakeTensorMap), and the pipe (barrier
// ring) the copies signal.
template <class GlobalTile, class Subj, class PipeTag>
struct TmaTiled {
    using global_tile = GlobalTile;
    using subject = Subj;
    using pipe = PipeTag;
};

template <class Pattern, class Elem, int TileK, class Cap, bool RowMajor>
struct select_swizzle {
    using type = axp::swizzle::None;
};
template <class Elem, int TileK, class Cap, bool RowMajor>
struct select_swizzle<axp::intent::memory_pattern::Optimized, Elem, TileK, Cap, RowMajor> {
    static constexpr int row_bytes = Elem::bytes * TileK;
    using type = std::conditional_t<
        Cap::has_tma && (row_bytes >= 128), axp::swizzle::B128,
        std::conditional_t<Cap::has_tma && (row_bytes >= 64), axp::swizzle::B64,
                           std::conditional_t<Cap::has_tma && (row_bytes >= 32), axp::swizzle::B32, axp::swizzle::None>>>;
};

template <class LoadMode, class Cap, class GlobalTile, class Subj, class PipeTag>
struct select_tma {
    using type = void;
};
template <class Cap, class GlobalTile, class Subj, class PipeTag>
struct select_tma<axp::intent::load_mode::AsyncPrefetch, Cap, GlobalTile, Subj, PipeTag> {
    using type = std::conditional_t<Cap::has_tma, TmaTiled<GlobalTile, Subj, PipeTag>, void>;
};
template <class Cap, class GlobalTile, class Subj, class PipeTag>
struct select_tma<axp::intent::load_mode::Streaming, Cap, GlobalTile, Subj, PipeTag> {
    using type = streaming_tag;
};
template <class Cap, class GlobalTile, class Subj, class PipeTag>
struct select_tma<axp::intent::load_mode::DeterministicLatency, Cap, GlobalTile, Subj, PipeTag> {
    using type = streaming_tag;
};

template <class Schedule, class Cap>
struct select_schedule {
    using type = Schedule;
};
template <class Cap>
struct select_schedule<axp::intent::schedule::ProducerConsumer, Cap> {
    static_assert(Cap::has_wgmma || Cap::has_tcgen05, "ProducerConsumer schedule requires a target with an asynchronous MMA unit");
    using type = axp::intent::schedule::ProducerConsumer;
};

}  // namespace axp::kit::detail

namespace axp::kit::expert {

// Specialise to force a choice; `void` means "no override".
template <class Pattern, class Elem, int TileK, class Cap, bool RowMajor>
struct swizzle_override {
    using type = void;
};
template <class LoadMode, class Cap, class GlobalTile, class Subj, class PipeTag>
struct tma_override {
    using type = void;
};
template <class Schedule, class Cap>
struct schedule_override {
    using type = void;
};

}  // namespace axp::kit::expert

namespace axp::kit::detail {

template <class Override, class Base>
using override_or_t = std::conditional_t<!std::is_void_v<Override>, Override, Base>;

template <class Pattern, class Elem, int TileK, class Cap, bool RowMajor>
using select_swizzle_t = override_or_t<typename axp::kit::expert::swizzle_override<Pattern, Elem, TileK, Cap, RowMajor>::type,
                                       typename select_swizzle<Pattern, Elem, TileK, Cap, RowMajor>::type>;

template <class LoadMode, class Cap, class GlobalTile, class Subj, class PipeTag>
using select_tma_t = override_or_t<typename axp::kit::expert::tma_override<LoadMode, Cap, GlobalTile, Subj, PipeTag>::type,
                                   typename select_tma<LoadMode, Cap, GlobalTile, Subj, PipeTag>::type>;

template <class Schedule, class Cap>
using select_schedule_t = override_or_t<typename axp::kit::expert::schedule_override<Schedule, Cap>::type,
                                        typename select_schedule<Schedule, Cap>::type>;

template <class T>
inline constexpr bool is_tma_config_v = false;
template <class G, class S, class P>
inline constexpr bool is_tma_config_v<TmaTiled<G, S, P>> = true;

}  // namespace axp::kit::detail
