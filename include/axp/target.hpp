// Compile-time target capability (reference include/axp/target.hpp:7-38): device
// passes use __CUDA_ARCH__, host passes need AXP_TARGET_SM; sm100 additionally
// needs AXP_ENABLE_SM100.  Only the sm90 and sm100 lanes exist in this tree.
// Public surface restated from tribe-iro/iro-cuda-ax (MIT licence, Copyright (c) 2026 IRO; the notice is kept in
// THIRD_PARTY_NOTICES.md at the repository root).
#pragma once
#include <iro_cuda_ax_core.hpp>

#if defined(__CUDA_ARCH__)
#undef AXP_TARGET_SM
#define AXP_TARGET_SM __CUDA_ARCH__
#elif !defined(AXP_TARGET_SM)
#error "AXP_TARGET_SM must be defined for host compilation (expected 900 or 1000)."
#endif

namespace axp {
#if AXP_TARGET_SM >= 1000
#ifdef AXP_ENABLE_SM100
using target_cap = iro::cap::sm100;
#else
static_assert(AXP_TARGET_SM < 1000, "AXP target selects SM100 but AXP_ENABLE_SM100 is not defined.");
#endif
#elif AXP_TARGET_SM >= 900
using target_cap = iro::cap::sm90;
#else
static_assert(AXP_TARGET_SM >= 900, "Unsupported AXP_TARGET_SM.");
#endif
}  // namespace axp
