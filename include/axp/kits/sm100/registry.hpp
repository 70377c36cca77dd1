// sm100 kit: obligation -> realization table.  The reference ships this file with
// a static_assert "no SM100 realizations are registered"
// (include/axp/kits/sm100/registry.hpp:10-14); the sm90 table it would mirror is
// include/axp/kits/sm90/registry.hpp:50-60,89-98.
//
// A registration names the leaf structs of include/axp/realize/sm100.hpp whose
// execute() members carry the device code for that obligation.
#pragma once
#include <iro_cuda_ax_core.hpp>

#include "../../protocol/sm100_contracts.hpp"
#include "../../realize/sm100.hpp"
#include "../../realize/sm100_host.hpp"
#include "../../realize/sm100_mask.hpp"

namespace axp::kit::sm100 {

namespace px = axp::protocol::sm100;
namespace rz = axp::realize::sm100;
using iro::bind::RealizationEntry;
using iro::util::fnv1a_64_cstr;
using iro::util::type_list;

// A realization: the obligation it discharges, an implementation id, and the leaf
// structs (with execute()) it is made of.
template <class O, iro::util::u64 ImplId, class... Leaves>
struct Realized : iro::contract::Realization<O, ImplId> {
    using leaves = type_list<Leaves...>;
};

template <class O>
struct registry_for {
    static_assert(sizeof(O) == 0, "axp::kit::sm100: no realization registered for this obligation");
};

#define AXP_SM100_REGISTER(TEMPLATE_HEAD, OBLIGATION, IMPL_NAME, ...)                                              \
    TEMPLATE_HEAD struct registry_for<OBLIGATION> {                                                                \
        using realization = Realized<OBLIGATION, fnv1a_64_cstr("axp.realize.sm100." IMPL_NAME) __VA_OPT__(, ) __VA_ARGS__>; \
        using type = type_list<RealizationEntry<realization, iro::cap::sm100>>;                                    \
    }

#define AXP_T(...) template <__VA_ARGS__>
#define AXP_O(...) __VA_ARGS__

// Every leaf carries its code in a member named `execute` (possibly overloaded or a template).  Detection by name:
// a class that inherits both the leaf and a fallback with a data member `execute` makes `&D::execute` ambiguous
// exactly when the leaf has a member of that name.
namespace detail {
struct execute_fallback {
    int execute;
};
template <class L>
struct execute_probe : L, execute_fallback {};
template <class L, class = void>
struct has_execute : std::true_type {};
template <class L>
struct has_execute<L, std::void_t<decltype(&execute_probe<L>::execute)>> : std::false_type {};
template <class List>
struct all_have_execute;
template <class... Ls>
struct all_have_execute<type_list<Ls...>> : std::bool_constant<(sizeof...(Ls) > 0) && (has_execute<Ls>::value && ...)> {};
}  // namespace detail

#if defined(__CUDACC__)
AXP_SM100_REGISTER(AXP_T(class S, class E, int R), AXP_O(px::HostMakeTensorMap<S, E, R>), "tma.host_make_tensor_map",
                   rz::HostTensorMapEncoder);
AXP_SM100_REGISTER(AXP_T(class S, int B, int N, int G), AXP_O(px::StageRing<S, B, N, 2, G>), "stage.ring_2d", rz::BarrierInit,
                   rz::BarrierExpectTx, rz::BulkTmaCopy2D, rz::BarrierWait, rz::MakeSmemDescKMajorSw128);
AXP_SM100_REGISTER(AXP_T(class S, int B, int N, int G), AXP_O(px::StageRing<S, B, N, 3, G>), "stage.ring_3d", rz::BarrierInit,
                   rz::BarrierExpectTx, rz::BulkTmaCopy3D, rz::BarrierWait, rz::MakeSmemDescKMajorSw128,
                   rz::MakeSmemDescMnMajorSw128);
AXP_SM100_REGISTER(template <>, px::BoundedBarrierWait, "sync.bounded_wait", rz::BarrierTryWait, rz::BarrierWait);
AXP_SM100_REGISTER(AXP_T(int C, int G), AXP_O(px::TmemAllocate<C, G>), "tmem.alloc", rz::TmemAlloc<G>);
AXP_SM100_REGISTER(AXP_T(int C, int G), AXP_O(px::TmemRelease<C, G>), "tmem.dealloc", rz::TmemDealloc<G>);
AXP_SM100_REGISTER(AXP_T(int M, int N, int K, class EA, class EB, int G, px::Major BM, class SA, class SB, class SD),
                   AXP_O(px::Tcgen05Mma<M, N, K, EA, EB, G, px::OperandSource::shared, BM, SA, SB, SD>), "compute.tcgen05_mma_ss",
                   rz::Tcgen05Mma<G, (EA::bytes == 2)>, rz::Tcgen05FenceAfter);
AXP_SM100_REGISTER(AXP_T(int M, int N, int K, class EA, class EB, px::Major BM, class SA, class SB, class SD),
                   AXP_O(px::Tcgen05Mma<M, N, K, EA, EB, 1, px::OperandSource::tmem, BM, SA, SB, SD>), "compute.tcgen05_mma_ts",
                   rz::Tcgen05MmaTmemA<(EA::bytes == 2)>, rz::Tcgen05FenceAfter);
AXP_SM100_REGISTER(AXP_T(int G, class S), AXP_O(px::Tcgen05Commit<G, S>), "compute.tcgen05_commit", rz::Tcgen05Commit<G>);
AXP_SM100_REGISTER(AXP_T(int C, class S), AXP_O(px::TmemToRegisters<C, S>), "tmem.ld_32x32b", rz::TmemLoad32x32, rz::TmemLoadWait,
                   rz::Tcgen05FenceBefore);
AXP_SM100_REGISTER(AXP_T(int C, class S), AXP_O(px::RegistersToTmem<C, S>), "tmem.st_32x32b", rz::TmemStore32x32, rz::TmemStoreWait,
                   rz::Tcgen05FenceBefore);
AXP_SM100_REGISTER(AXP_T(int B, int N, class S), AXP_O(px::RegistersToSharedOperand<B, N, S>), "stage.registers_to_shared_operand", rz::AsyncProxyFence,
                   rz::BarrierArrive, rz::MakeSmemDescKMajorSw128);
AXP_SM100_REGISTER(AXP_T(class R, class S, class SA, class SB), AXP_O(px::ScalePromoteAccumulator<R, S, SA, SB>), "scale.promote_fma", rz::ScalePromoteFma);
AXP_SM100_REGISTER(AXP_T(class P, class SI, class SO), AXP_O(px::CastPack<iro::elem::f32, iro::elem::bf16, P, SI, SO>), "convert.pack_bf16x2",
                   rz::PackBf16x2);
AXP_SM100_REGISTER(AXP_T(class P, class SI, class SO), AXP_O(px::CastPack<iro::elem::f32, iro::elem::e4m3, P, SI, SO>), "convert.pack_e4m3x4_sat",
                   rz::PackE4m3x4);
AXP_SM100_REGISTER(AXP_T(class P, class S), AXP_O(px::CastWeights<iro::elem::bf16, P, S>), "convert.weights_bf16x2", rz::PackBf16x2);
AXP_SM100_REGISTER(AXP_T(class P, class S), AXP_O(px::CastWeights<iro::elem::e4m3, P, S>), "convert.weights_e4m3x4_sat", rz::PackE4m3x4);
AXP_SM100_REGISTER(AXP_T(class B, class A, class S), AXP_O(px::BiasActivation<B, A, S>), "epilogue.bias_activation", rz::BiasActFma);
AXP_SM100_REGISTER(AXP_T(class U, class A, class S), AXP_O(px::GatedActivation<U, A, S>), "epilogue.gated_activation", rz::BiasActFma);
AXP_SM100_REGISTER(AXP_T(class C, class A, class B, class S), AXP_O(px::LinearCombination<C, A, B, S>), "epilogue.linear_combination", rz::BiasActFma);
AXP_SM100_REGISTER(AXP_T(class E, class S), AXP_O(px::StoreRowGlobal<E, S>), "store.row_vec16", rz::RowStoreVec16);
AXP_SM100_REGISTER(AXP_T(int M, int N, class S), AXP_O(px::CausalMaskPredicate<M, N, S>), "mask.causal_pred", rz::CausalMaskPred);
AXP_SM100_REGISTER(AXP_T(class S, class P, class St), AXP_O(px::RowSoftmaxStateUpdateOn<S, P, St>), "softmax.row_state_exp2", rz::RowSoftmaxExp2);
AXP_SM100_REGISTER(AXP_T(class O_, class St), AXP_O(px::RescaleAccumulatorInTmemOn<O_, St>), "softmax.rescale_tmem", rz::TmemLoad32x32, rz::TmemStore32x32,
                   rz::TmemStoreWait);
AXP_SM100_REGISTER(AXP_T(int P, int M), AXP_O(px::RoleRegisterBudget<P, M>), "specialize.setmaxnreg", rz::RegDealloc<P>,
                   rz::RegAlloc<M>);
#endif

#undef AXP_SM100_REGISTER
#undef AXP_T
#undef AXP_O

template <class O>
using registry_for_t = typename registry_for<O>::type;

// Resolved<O, R> with R the realization that the sm100 capability gets for O
// (reference `axp::kit::sm100::bind`, include/axp/kits/sm100/registry.hpp:19-20).
template <class O>
using bind = iro::bind::lookup_realization_t<O, iro::cap::sm100, registry_for_t<O>>;

// every obligation of the list binds, and every leaf of every bound realization has an execute member
template <class List>
struct binds_all;
template <class... Os>
struct binds_all<type_list<Os...>>
    : std::bool_constant<((bind<Os>::found && detail::all_have_execute<typename bind<Os>::realization::leaves>::value) && ...)> {};

}  // namespace axp::kit::sm100
