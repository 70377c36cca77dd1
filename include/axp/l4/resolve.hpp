// (graph_hash, capability, profile) -> manifest row -> realization key and bind key
// (reference include/axp/l4/resolve.hpp:29-61, same checks in the same order).
// Public surface restated from tribe-iro/iro-cuda-ax (MIT licence, Copyright (c) 2026 IRO; the notice is kept in
// THIRD_PARTY_NOTICES.md at the repository root).
#pragma once

#if !defined(AXP_LIBRARY_BUILD)
#error "axp/l4/resolve.hpp is library-only; use axp/l4.hpp in application code."
#endif

#include "../graph/hash.hpp"
#include "../graph/verify.hpp"
#include "../l4.hpp"
#include "../level3/attention.hpp"
#include "../level3/gemm.hpp"
#include "../target.hpp"
#include "bind_key.hpp"
#include "lowering.hpp"
#include "graph_registry_index.hpp"

namespace axp::l4 {

namespace detail {
template <class Pattern, class = void>
struct has_lowering : std::false_type {};
template <class Pattern>
struct has_lowering<Pattern, std::void_t<axp::l4::lowering::to_l3_pattern_t<Pattern>>> : std::true_type {};
}  // namespace detail

template <class G, class Cap = axp::target_cap, class ProfileT = axp::l4::profile::proof_full>
struct resolve {
    static_assert(axp::graph::verify<G>(), "axp::l4::resolve: graph verification failed");

    static constexpr iro::util::u64 graph_hash = axp::graph::graph_hash_v<G>;
    using registry_entry = axp::l4::graph_registry::entry<graph_hash, Cap, ProfileT>;

    static_assert(registry_entry::enabled,
                  "axp::l4::resolve: no manifest-enabled graph row for (graph_hash, capability, profile)");
    static_assert(!std::is_same_v<typename registry_entry::pattern, void>, "axp::l4::resolve: registry row missing pattern type");
    static_assert(axp::l4::manifest::enabled_v<typename registry_entry::pattern, Cap>,
                  "axp::l4::resolve: pattern/capability pair is not manifest-enabled");

    using l4_pattern = typename registry_entry::pattern;
    static_assert(axp::l4::lowering::is_canonical_preset_pattern_v<l4_pattern>,
                  "axp::l4::resolve: registry pattern must be canonical axp::l4::preset::*");
    static_assert(detail::has_lowering<l4_pattern>::value, "axp::l4::resolve: missing L4->L3 lowering for registry pattern");
    using pattern = axp::l4::lowering::to_l3_pattern_t<l4_pattern>;
    using graph = axp::level3::registry::Select<pattern, Cap>;
    static constexpr iro::util::u64 realization_key = registry_entry::realization_key;
    static constexpr iro::util::u64 bind_key = axp::l4::bind_key_v<graph_hash, Cap, ProfileT, realization_key>;
    using type = graph;
};

template <class G, class Cap = axp::target_cap, class ProfileT = axp::l4::profile::proof_full>
using Select = typename resolve<G, Cap, ProfileT>::type;

template <class G, class Cap = axp::target_cap, class ProfileT = axp::l4::profile::proof_full>
struct supports : std::bool_constant<axp::l4::graph_registry::enabled_v<axp::graph::graph_hash_v<G>, Cap, ProfileT>> {};

}  // namespace axp::l4
