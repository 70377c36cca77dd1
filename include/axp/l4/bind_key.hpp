// Profiles and the bind key (reference include/axp/l4/bind_key.hpp:11-38): the same
// mixing order, so that a key computed here equals the reference's for the same
// (graph_hash, capability, profile, realization_key).
// Public surface restated from tribe-iro/iro-cuda-ax (MIT licence, Copyright (c) 2026 IRO; the notice is kept in
// THIRD_PARTY_NOTICES.md at the repository root).
#pragma once

#if !defined(AXP_LIBRARY_BUILD)
#error "axp/l4/bind_key.hpp is library-only; use axp/l4.hpp in application code."
#endif

#include <iro_cuda_ax_core.hpp>

namespace axp::l4::profile {
struct dev_fast { static constexpr iro::util::u64 id = iro::util::fnv1a_64_cstr("axp.l4.profile.dev_fast"); };
struct proof_full { static constexpr iro::util::u64 id = iro::util::fnv1a_64_cstr("axp.l4.profile.proof_full"); };
}  // namespace axp::l4::profile

namespace axp::l4 {

template <iro::util::u64 GraphHash, class Cap, class ProfileT, iro::util::u64 RealizationKey>
struct BindKey {
    static constexpr iro::util::u64 value = iro::util::mix_u64(
        iro::util::fnv1a_64_cstr("axp.l4.bind_key.v2"),
        iro::util::mix_u64(GraphHash, iro::util::mix_u64(Cap::id, iro::util::mix_u64(ProfileT::id, RealizationKey))));
};
template <iro::util::u64 GraphHash, class Cap, class ProfileT, iro::util::u64 RealizationKey>
inline constexpr iro::util::u64 bind_key_v = BindKey<GraphHash, Cap, ProfileT, RealizationKey>::value;

}  // namespace axp::l4
