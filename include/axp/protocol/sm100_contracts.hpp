// Obligations (contracts) of the sm100 gemm / attention graphs.  Each is a type
// with a stable id and the resources it holds; the sm100 kit maps every one to a
// realization with device code (include/axp/kits/sm100/registry.hpp).
//
// Reference vocabulary these stand for:
//   tensor maps / bulk copies   include/axp/protocol/tma/contracts.hpp:58-185
//   slot typestate + barriers   include/axp/protocol/stage/pipeline_contracts.hpp:31-90,
//                               include/axp/protocol/sync/contracts.hpp
//   Tcgen05Mma                  include/axp/protocol/compute/contracts.hpp:302-415
//   TileToTmem / TmemToTile     include/axp/protocol/tmem/contracts.hpp:21-132
//   CastTile                    include/axp/protocol/convert/contracts.hpp:31
//   ScaleSharedTile             include/axp/protocol/scale/contracts.hpp:21-68
//   CausalMask                  include/axp/level1/mask.hpp
// The reference keeps `is_tcgen05_shape_v` false for every shape
// (include/axp/protocol/compute/detail/mma_shapes.hpp:57-58); here it states the
// legal dense shapes of tcgen05.mma.
#pragma once
#include <iro_cuda_ax_core.hpp>

namespace axp::protocol::sm100 {

using iro::contract::Obligation;
using iro::contract::Resources;
using iro::util::fnv1a_64_cstr;
using iro::util::mix_u64;
using iro::util::u64;

constexpr u64 mix3(u64 a, u64 b, u64 c) { return mix_u64(mix_u64(a, b), c); }

// M x N x K per instruction; K covers 32 bytes of the operand row.
template <int M, int N, int K, int ElemBytes, int CtaGroup>
inline constexpr bool is_tcgen05_shape_v =
    (K * ElemBytes == 32) &&
    ((CtaGroup == 1 && ((M == 64 && N % 8 == 0) || (M == 128 && N % 16 == 0))) ||
     (CtaGroup == 2 && ((M == 128 && N % 16 == 0) || (M == 256 && N % 16 == 0)))) &&
    (N >= 16 && N <= 256);

// Host: encode a tiled tensor map (128-byte swizzle, zero fill) for `Subj`.
template <class Subj, class Elem, int Rank>
struct HostMakeTensorMap : Obligation<mix3(fnv1a_64_cstr("axp.protocol.tma.host_make_tensor_map"), Subj::id, Elem::id + Rank)> {
    using subject = Subj;
    using elem = Elem;
    static constexpr int rank = Rank;
};

// A ring of `Stages` shared-memory slots of `TileBytes`, filled by bulk tensor
// copies that signal a "full" mbarrier and released through an "empty" mbarrier
// (slot typestate free -> filling -> ready -> used).  One CTA is the only writer
// of its slots.
template <class Subj, int TileBytes, int Stages, int Rank>
struct StageRing : Obligation<mix3(fnv1a_64_cstr("axp.protocol.stage.ring"), Subj::id, u64(TileBytes) * 64 + Stages * 8 + Rank),
                              Resources<TileBytes * Stages, 0, 2 * Stages>> {
    using subject = Subj;
    static constexpr int tile_bytes = TileBytes;
    static constexpr int stages = Stages;
    static constexpr int rank = Rank;
    static_assert(TileBytes % 1024 == 0, "128-byte swizzled slots must be 1024-byte aligned");
};

// Every wait on an mbarrier is bounded: it gives up after a cycle limit, records
// a status word and lets the kernel unwind.
struct BoundedBarrierWait : Obligation<fnv1a_64_cstr("axp.protocol.sync.bounded_barrier_wait")> {};

template <int Columns, int CtaGroup>
struct TmemAllocate : Obligation<mix_u64(fnv1a_64_cstr("axp.protocol.tmem.allocate"), Columns * 4 + CtaGroup), Resources<0, Columns, 0>> {
    static_assert(Columns >= 32 && (Columns & (Columns - 1)) == 0 && Columns <= 512, "TMEM allocations are powers of two in [32,512]");
};
template <int Columns, int CtaGroup>
struct TmemRelease : Obligation<mix_u64(fnv1a_64_cstr("axp.protocol.tmem.release"), Columns * 4 + CtaGroup)> {};

enum class OperandSource { shared, tmem };
enum class Major { k, mn };

// D[tmem, M x N fp32] (+)= A[M x K] . B[K x N], operands described by shared-memory
// matrix descriptors (or A in tensor memory), issued by one thread.
template <int M, int N, int K, class ElemA, class ElemB, int CtaGroup, OperandSource ASrc = OperandSource::shared,
          Major BMajor = Major::k>
struct Tcgen05Mma : Obligation<mix3(fnv1a_64_cstr("axp.protocol.compute.tcgen05_mma"), mix_u64(ElemA::id, ElemB::id),
                                    u64(M) * 1000003 + N * 1009 + K * 31 + CtaGroup * 7 + int(ASrc) * 3 + int(BMajor))> {
    static_assert(ElemA::bytes == ElemB::bytes, "tcgen05 operands of one instruction share a kind");
    static_assert(is_tcgen05_shape_v<M, N, K, ElemA::bytes, CtaGroup>, "not a tcgen05.mma shape");
    static constexpr int m = M, n = N, k = K, cta_group = CtaGroup;
};

// Arrive on an mbarrier when all previously issued MMAs have completed.
template <int CtaGroup>
struct Tcgen05Commit : Obligation<mix_u64(fnv1a_64_cstr("axp.protocol.compute.tcgen05_commit"), CtaGroup), Resources<0, 0, 1>> {};

template <int Columns>
struct TmemToRegisters : Obligation<mix_u64(fnv1a_64_cstr("axp.protocol.tmem.to_registers"), Columns)> {};
template <int Columns>
struct RegistersToTmem : Obligation<mix_u64(fnv1a_64_cstr("axp.protocol.tmem.from_registers"), Columns)> {};

// acc[m, n] += sA[m, kb] * sB[n / 128, kb] * partial[m, n]: the block scales are
// applied to the fp32 partial sum of one 128-wide K block (the reference's
// ScaleSharedTile re-quantises the operand in shared memory instead, which loses
// precision for fp8).
template <class Recipe>
struct ScalePromoteAccumulator : Obligation<mix_u64(fnv1a_64_cstr("axp.protocol.scale.promote_accumulator"), Recipe::id)> {
    static_assert(Recipe::has_scales, "scale promotion needs a recipe with operand scales");
};

template <class From, class To, class Policy>
struct CastPack : Obligation<mix3(fnv1a_64_cstr("axp.protocol.convert.cast_pack"), mix_u64(From::id, To::id), Policy::id)> {};

// Softmax weights P: fp32 -> operand element type (bf16, or E4M3 with saturation),
// written to tensor memory as the A operand of the PV MMA (reference CastWeights,
// include/axp/level3/recipes/attention/process.hpp:1594-1606).
template <class To, class Policy>
struct CastWeights : Obligation<mix3(fnv1a_64_cstr("axp.protocol.convert.cast_weights"), To::id, Policy::id)> {};

// Fused epilogue on the fp32 accumulator: out = Act(acc + bias[column]) (reference
// epilogue::BiasActivationVec, include/axp/level3/gemm.hpp:159-219).
// Act is one of axp::level3::epilogue::act::{Identity, SiLU}.
template <class BiasSubj, class Act>
struct BiasActivation : Obligation<mix3(fnv1a_64_cstr("axp.protocol.epilogue.bias_activation"), BiasSubj::id, Act::id)> {
    using bias_subject = BiasSubj;
    using activation = Act;
};

// out = Act(acc[:, n]) * acc[:, n + N/2]: the accumulator holds a "gate" and an "up" product of the same output
// columns side by side (the B tile is half gate rows, half up rows).
template <class UpSubj, class Act>
struct GatedActivation : Obligation<mix3(fnv1a_64_cstr("axp.protocol.epilogue.gated_activation"), UpSubj::id, Act::id)> {
    using up_subject = UpSubj;
    using activation = Act;
};

// out = (alpha * acc) + (beta * c): MulAcc, MulC and Add of the reference's LinearCombinationVec as three fp32
// operations on the accumulator fragment (include/axp/level3/gemm.hpp:187-208).
template <class CSubj, class AlphaSubj, class BetaSubj>
struct LinearCombination
    : Obligation<mix3(fnv1a_64_cstr("axp.protocol.epilogue.linear_combination"), CSubj::id, mix_u64(AlphaSubj::id, BetaSubj::id))> {
    using c_subject = CSubj;
    using alpha_subject = AlphaSubj;
    using beta_subject = BetaSubj;
};

// Registers -> a 128-byte-swizzled operand tile in shared memory (`Slots` tiles of `TileBytes`), made visible to the
// tensor core with a proxy fence: the route of the E4M3 softmax weights P to the P.V MMA (the S region in tensor memory
// is then free as soon as the softmax holds it in registers).
template <int TileBytes, int Slots>
struct RegistersToSharedOperand : Obligation<mix_u64(fnv1a_64_cstr("axp.protocol.stage.registers_to_shared_operand"), u64(TileBytes) * 16 + Slots),
                                             Resources<TileBytes * Slots, 0, Slots>> {
    static_assert(TileBytes % 1024 == 0, "128-byte swizzled tiles must be 1024-byte aligned");
};

template <class Elem>
struct StoreRowGlobal : Obligation<mix_u64(fnv1a_64_cstr("axp.protocol.store.row_global"), Elem::id)> {};

// valid = (k_base + col) <= (q_base + row); whole tile skipped when k_base > q_base + TileM - 1.
template <int TileM, int TileN>
struct CausalMaskPredicate : Obligation<mix_u64(fnv1a_64_cstr("axp.protocol.mask.causal"), TileM * 4096 + TileN)> {};

// Per-row online softmax: m' = max(m, rowmax), l' = l*exp(m-m') + rowsum(exp(s-m')).
struct RowSoftmaxStateUpdate : Obligation<fnv1a_64_cstr("axp.protocol.softmax.row_state_update")> {};
// acc *= exp(m - m') in tensor memory, only when the row maximum grew.
struct RescaleAccumulatorInTmem : Obligation<fnv1a_64_cstr("axp.protocol.softmax.rescale_accumulator_tmem")> {};

// Register budget moved from the producer / MMA warpgroup to the math warpgroups.
template <int ProducerRegs, int MathRegs>
struct RoleRegisterBudget : Obligation<mix_u64(fnv1a_64_cstr("axp.protocol.specialize.register_budget"), ProducerRegs * 1024 + MathRegs)> {
    static constexpr int producer_regs = ProducerRegs, math_regs = MathRegs;
};

}  // namespace axp::protocol::sm100
