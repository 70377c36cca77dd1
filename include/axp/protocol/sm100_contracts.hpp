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
//
// Ports.  Every obligation that moves or makes data names what it needs and what it leaves behind as token lists on
// input / output ports (reference: iro::contract::InputPort / OutputPort, checked by
// axp::protocol::audit::contract_tokens_complete, include/axp/protocol/audit/tokens.hpp:35-80).  Subjects are wires
// placed in a memory space (axp::subject::at<space, wire>): a copy or an MMA reads a wire in one space and provides it
// (or its result) in another.  Two facts of the sm_100a execution model are written into the tokens:
//   * a tcgen05.mma leaves its accumulator visible to the issuing thread's later tcgen05 instructions only
//     (visible_at<.., scope::lane>); the tcgen05.commit that follows is what publishes it to the CTA (pair) together
//     with the mbarrier phase the readers wait on (visible_at + sync_at at block / cluster scope);
//   * data written to tensor memory or shared memory by the softmax warps for the tensor core (P, the rescaled O) is
//     published by the mbarrier hand-over that follows the store and its fence (sync_at<.., scope::block>).
// axp::graph::flow_closed walks a graph's obligation list and checks that every required token is provided earlier
// (include/axp/graph/flow.hpp).
#pragma once
#include <iro_cuda_ax_core.hpp>

#include "../bundles/token_bundles.hpp"
#include "../naming/subjects.hpp"

namespace axp::protocol::sm100 {

using iro::contract::Obligation;
using iro::contract::Resources;
using iro::util::fnv1a_64_cstr;
using iro::util::mix_u64;
using iro::util::type_list;
using iro::util::u64;

constexpr u64 mix3(u64 a, u64 b, u64 c) { return mix_u64(mix_u64(a, b), c); }

// ---- port shorthands ----
namespace ex = iro::exec;
namespace life = iro::token::lifetime;
namespace sp = iro::contract::space;
namespace sj = axp::subject;
// the tensor-core executor of a CTA group and the lifetime of what it shares
template <int CtaGroup>
using cta_exec = std::conditional_t<CtaGroup == 2, ex::cta_group2, ex::cta_group1>;
template <int CtaGroup>
using cta_life = std::conditional_t<CtaGroup == 2, life::cluster, life::block>;
// a tile that `Exec` reads / has written; `Placed` is an axp::subject::at<space, wire>
template <class Placed, class Exec, class Lifetime>
using tile_in = iro::contract::InputPort<iro::contract::Tile<typename Placed::space>, Placed, Exec, axp::bundle::TileInTokens<Placed, Exec, Lifetime>>;
template <class Placed, class Exec, class Lifetime>
using tile_out = iro::contract::OutputPort<iro::contract::Tile<typename Placed::space>, Placed, Exec, axp::bundle::TileOutTokens<Placed, Exec, Lifetime>>;
template <class Subj, class Exec, class Lifetime>
using handle_in = iro::contract::InputPort<iro::contract::Handle, Subj, Exec, axp::bundle::ValueLive<Subj, Lifetime>>;
template <class Subj, class Exec, class Lifetime>
using handle_out = iro::contract::OutputPort<iro::contract::Handle, Subj, Exec, axp::bundle::ValueLive<Subj, Lifetime>>;
template <class Subj, class Exec, class Lifetime>
using scalar_in = iro::contract::InputPort<iro::contract::Scalar, Subj, Exec, axp::bundle::ValueLive<Subj, Lifetime>>;
template <class Subj, class Exec, class Lifetime>
using scalar_out = iro::contract::OutputPort<iro::contract::Scalar, Subj, Exec, axp::bundle::ValueLive<Subj, Lifetime>>;
// a register fragment of one warp
template <class Subj>
using frag_in = tile_in<sj::in_regs<Subj>, ex::warp, life::warp>;
template <class Subj>
using frag_out = tile_out<sj::in_regs<Subj>, ex::warp, life::warp>;
// a global tensor read by single threads of the kernel (scales, bias, C)
template <class Subj>
using global_in = tile_in<sj::in_global<Subj>, ex::lane, life::kernel>;

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
    using inputs = type_list<tile_in<sj::in_global<Subj>, ex::host, life::kernel>>;
    using outputs = type_list<handle_out<sj::tensor_map_of<Subj>, ex::host, life::kernel>>;
};

// A ring of `Stages` shared-memory slots of `TileBytes`, filled by bulk tensor
// copies that signal a "full" mbarrier and released through an "empty" mbarrier
// (slot typestate free -> filling -> ready -> used).  One CTA is the only writer
// of its slots.  CtaGroup = 2: the leader's "full" barrier counts the bytes of both CTAs of the pair, so a completed
// phase publishes the pair's tiles at cluster scope.
template <class Subj, int TileBytes, int Stages, int Rank, int CtaGroup = 1>
struct StageRing : Obligation<mix3(fnv1a_64_cstr("axp.protocol.stage.ring"), Subj::id, u64(TileBytes) * 64 + Stages * 8 + Rank + u64(CtaGroup - 1) * 4),
                              Resources<TileBytes * Stages, 0, 2 * Stages>> {
    using subject = Subj;
    static constexpr int tile_bytes = TileBytes;
    static constexpr int stages = Stages;
    static constexpr int rank = Rank;
    static constexpr int cta_group = CtaGroup;
    static_assert(TileBytes % 1024 == 0, "128-byte swizzled slots must be 1024-byte aligned");
    // one elected thread issues the copies from the global tensor through its tensor map
    using inputs = type_list<handle_in<sj::tensor_map_of<Subj>, ex::lane, life::kernel>, global_in<Subj>>;
    // the completed "full" phase publishes the slot to the tensor core of the CTA (pair)
    using outputs = type_list<tile_out<sj::in_shared<Subj>, cta_exec<CtaGroup>, cta_life<CtaGroup>>>;
};

// Every wait on an mbarrier is bounded: it gives up after a cycle limit, records
// a status word and lets the kernel unwind.
struct BoundedBarrierWait : Obligation<fnv1a_64_cstr("axp.protocol.sync.bounded_barrier_wait")> {};

template <int Columns, int CtaGroup>
struct TmemAllocate : Obligation<mix_u64(fnv1a_64_cstr("axp.protocol.tmem.allocate"), Columns * 4 + CtaGroup), Resources<0, Columns, 0>> {
    static_assert(Columns >= 32 && (Columns & (Columns - 1)) == 0 && Columns <= 512, "TMEM allocations are powers of two in [32,512]");
    using outputs = type_list<handle_out<sj::tmem_base, ex::warp, cta_life<CtaGroup>>>;
};
template <int Columns, int CtaGroup>
struct TmemRelease : Obligation<mix_u64(fnv1a_64_cstr("axp.protocol.tmem.release"), Columns * 4 + CtaGroup)> {
    using inputs = type_list<handle_in<sj::tmem_base, ex::warp, cta_life<CtaGroup>>>;
};

enum class OperandSource { shared, tmem };
enum class Major { k, mn };

// D[tmem, M x N fp32] (+)= A[M x K] . B[K x N], operands described by shared-memory
// matrix descriptors (or A in tensor memory), issued by one thread.
// ASubj / BSubj / DSubj are the wires of the operands and of the accumulator; A sits in shared memory or, for
// OperandSource::tmem, in tensor memory.
template <int M, int N, int K, class ElemA, class ElemB, int CtaGroup, OperandSource ASrc = OperandSource::shared,
          Major BMajor = Major::k, class ASubj = sj::MatrixA, class BSubj = sj::MatrixB, class DSubj = sj::Accumulator>
struct Tcgen05Mma : Obligation<mix3(mix3(fnv1a_64_cstr("axp.protocol.compute.tcgen05_mma"), ASubj::id, mix_u64(BSubj::id, DSubj::id)),
                                    mix_u64(ElemA::id, ElemB::id),
                                    u64(M) * 1000003 + N * 1009 + K * 31 + CtaGroup * 7 + int(ASrc) * 3 + int(BMajor))> {
    static_assert(ElemA::bytes == ElemB::bytes, "tcgen05 operands of one instruction share a kind");
    static_assert(is_tcgen05_shape_v<M, N, K, ElemA::bytes, CtaGroup>, "not a tcgen05.mma shape");
    static constexpr int m = M, n = N, k = K, cta_group = CtaGroup;
    using a_placed = std::conditional_t<ASrc == OperandSource::tmem, sj::in_tmem<ASubj>, sj::in_shared<ASubj>>;
    // the tensor core of the CTA (pair) reads the operands: they must have been published at that scope
    using inputs = type_list<tile_in<a_placed, cta_exec<CtaGroup>, cta_life<CtaGroup>>,
                             tile_in<sj::in_shared<BSubj>, cta_exec<CtaGroup>, cta_life<CtaGroup>>,
                             handle_in<sj::tmem_base, ex::lane, cta_life<CtaGroup>>>;
    // issued, not yet published: only the issuing thread's later tcgen05 instructions are ordered after it
    using outputs = type_list<tile_out<sj::in_tmem<DSubj>, ex::lane, cta_life<CtaGroup>>>;
};

// Arrive on an mbarrier when all previously issued MMAs have completed.
// `Subj` is the accumulator wire whose MMAs the commit covers: the completed mbarrier phase publishes it.
template <int CtaGroup, class Subj = sj::Accumulator>
struct Tcgen05Commit : Obligation<mix3(fnv1a_64_cstr("axp.protocol.compute.tcgen05_commit"), Subj::id, CtaGroup), Resources<0, 0, 1>> {
    using inputs = type_list<tile_in<sj::in_tmem<Subj>, ex::lane, cta_life<CtaGroup>>>;
    using outputs = type_list<tile_out<sj::in_tmem<Subj>, cta_exec<CtaGroup>, cta_life<CtaGroup>>>;
};

// tcgen05.ld 32x32b: a warp reads `Columns` columns of its 32 tensor-memory lanes into registers.
template <int Columns, class Subj = sj::Accumulator>
struct TmemToRegisters : Obligation<mix3(fnv1a_64_cstr("axp.protocol.tmem.to_registers"), Subj::id, Columns)> {
    using inputs = type_list<tile_in<sj::in_tmem<Subj>, ex::warp, life::warp>>;
    using outputs = type_list<frag_out<Subj>>;
};
// tcgen05.st 32x32b + wait + fence + the mbarrier hand-over to the issuing thread: the warpgroup's rows of `Subj` in
// tensor memory, published to the CTA.
template <int Columns, class Subj = sj::AttentionP>
struct RegistersToTmem : Obligation<mix3(fnv1a_64_cstr("axp.protocol.tmem.from_registers"), Subj::id, Columns)> {
    using inputs = type_list<frag_in<Subj>, handle_in<sj::tmem_base, ex::warp, life::block>>;
    using outputs = type_list<tile_out<sj::in_tmem<Subj>, ex::cta_group1, life::block>>;
};

// acc[m, n] += sA[m, kb] * sB[n / 128, kb] * partial[m, n]: the block scales are
// applied to the fp32 partial sum of one 128-wide K block (the reference's
// ScaleSharedTile re-quantises the operand in shared memory instead, which loses
// precision for fp8).
template <class Recipe, class AccSubj = sj::Accumulator, class ScaleASubj = sj::ScaleA, class ScaleBSubj = sj::ScaleB>
struct ScalePromoteAccumulator : Obligation<mix3(mix_u64(fnv1a_64_cstr("axp.protocol.scale.promote_accumulator"), Recipe::id), AccSubj::id,
                                                 mix_u64(ScaleASubj::id, ScaleBSubj::id))> {
    static_assert(Recipe::has_scales, "scale promotion needs a recipe with operand scales");
    using inputs = type_list<frag_in<AccSubj>, global_in<ScaleASubj>, global_in<ScaleBSubj>>;
    using outputs = type_list<frag_out<AccSubj>>;
};

// fp32 fragment of `InSubj` -> packed `To` fragment of `OutSubj`
template <class From, class To, class Policy, class InSubj = sj::Accumulator, class OutSubj = sj::MatrixC>
struct CastPack : Obligation<mix3(mix3(fnv1a_64_cstr("axp.protocol.convert.cast_pack"), InSubj::id, OutSubj::id), mix_u64(From::id, To::id), Policy::id)> {
    using inputs = type_list<frag_in<InSubj>>;
    using outputs = type_list<frag_out<OutSubj>>;
};

// Softmax weights P: fp32 -> operand element type (bf16, or E4M3 with saturation),
// written to tensor memory as the A operand of the PV MMA (reference CastWeights,
// include/axp/level3/recipes/attention/process.hpp:1594-1606).
template <class To, class Policy, class PSubj = sj::AttentionP>
struct CastWeights : Obligation<mix3(mix_u64(fnv1a_64_cstr("axp.protocol.convert.cast_weights"), PSubj::id), To::id, Policy::id)> {
    using inputs = type_list<frag_in<PSubj>>;
    using outputs = type_list<frag_out<PSubj>>;
};

// Fused epilogue on the fp32 accumulator: out = Act(acc + bias[column]) (reference
// epilogue::BiasActivationVec, include/axp/level3/gemm.hpp:159-219).
// Act is one of axp::level3::epilogue::act::{Identity, SiLU}.
template <class BiasSubj, class Act, class AccSubj = sj::Accumulator>
struct BiasActivation : Obligation<mix3(mix_u64(fnv1a_64_cstr("axp.protocol.epilogue.bias_activation"), AccSubj::id), BiasSubj::id, Act::id)> {
    using bias_subject = BiasSubj;
    using activation = Act;
    using inputs = type_list<frag_in<AccSubj>, global_in<BiasSubj>>;
    using outputs = type_list<frag_out<AccSubj>>;
};

// out = Act(acc[:, n]) * acc[:, n + N/2]: the accumulator holds a "gate" and an "up" product of the same output
// columns side by side (the B tile is half gate rows, half up rows).
template <class UpSubj, class Act, class AccSubj = sj::Accumulator>
struct GatedActivation : Obligation<mix3(mix_u64(fnv1a_64_cstr("axp.protocol.epilogue.gated_activation"), AccSubj::id), UpSubj::id, Act::id)> {
    using up_subject = UpSubj;
    using activation = Act;
    // gate and up halves arrive in the same accumulator fragment
    using inputs = type_list<frag_in<AccSubj>>;
    using outputs = type_list<frag_out<AccSubj>>;
};

// out = (alpha * acc) + (beta * c): MulAcc, MulC and Add of the reference's LinearCombinationVec as three fp32
// operations on the accumulator fragment (include/axp/level3/gemm.hpp:187-208).
template <class CSubj, class AlphaSubj, class BetaSubj, class AccSubj = sj::Accumulator>
struct LinearCombination
    : Obligation<mix3(mix_u64(fnv1a_64_cstr("axp.protocol.epilogue.linear_combination"), AccSubj::id), CSubj::id, mix_u64(AlphaSubj::id, BetaSubj::id))> {
    using c_subject = CSubj;
    using alpha_subject = AlphaSubj;
    using beta_subject = BetaSubj;
    using inputs = type_list<frag_in<AccSubj>, global_in<CSubj>, scalar_in<AlphaSubj, ex::lane, life::kernel>,
                             scalar_in<BetaSubj, ex::lane, life::kernel>>;
    using outputs = type_list<frag_out<AccSubj>>;
};

// Registers -> a 128-byte-swizzled operand tile in shared memory (`Slots` tiles of `TileBytes`), made visible to the
// tensor core with a proxy fence: the route of the E4M3 softmax weights P to the P.V MMA (the S region in tensor memory
// is then free as soon as the softmax holds it in registers).
template <int TileBytes, int Slots, class Subj = sj::AttentionP>
struct RegistersToSharedOperand : Obligation<mix3(fnv1a_64_cstr("axp.protocol.stage.registers_to_shared_operand"), Subj::id, u64(TileBytes) * 16 + Slots),
                                             Resources<TileBytes * Slots, 0, Slots>> {
    static_assert(TileBytes % 1024 == 0, "128-byte swizzled tiles must be 1024-byte aligned");
    using inputs = type_list<frag_in<Subj>>;
    using outputs = type_list<tile_out<sj::in_shared<Subj>, ex::cta_group1, life::block>>;
};

// packed fragment of `Subj` -> rows of the global tensor `Subj`; plain stores, visible to the device when the kernel ends
template <class Elem, class Subj = sj::MatrixC>
struct StoreRowGlobal : Obligation<mix3(fnv1a_64_cstr("axp.protocol.store.row_global"), Subj::id, Elem::id)> {
    using inputs = type_list<frag_in<Subj>>;
    using outputs = type_list<tile_out<sj::in_global<Subj>, ex::warp, life::kernel>>;
};

// valid = (k_base + col) <= (q_base + row); whole tile skipped when k_base > q_base + TileM - 1.
template <int TileM, int TileN, class SSubj = sj::AttentionS>
struct CausalMaskPredicate : Obligation<mix3(fnv1a_64_cstr("axp.protocol.mask.causal"), SSubj::id, TileM * 4096 + TileN)> {
    using inputs = type_list<frag_in<SSubj>>;
    using outputs = type_list<frag_out<SSubj>>;
};

// Per-row online softmax: m' = max(m, rowmax), l' = l*exp(m-m') + rowsum(exp(s-m')).
// Scores of `SSubj` in registers -> unnormalised weights of `PSubj` in registers; the per-row state (m, l) is carried
// from step to step in registers of the row's thread.
template <class SSubj = sj::AttentionS, class PSubj = sj::AttentionP, class StateSubj = sj::SoftmaxState>
struct RowSoftmaxStateUpdateOn : Obligation<mix3(fnv1a_64_cstr("axp.protocol.softmax.row_state_update"), SSubj::id, mix_u64(PSubj::id, StateSubj::id))> {
    using inputs = type_list<frag_in<SSubj>, scalar_in<StateSubj, ex::lane, life::warp>>;
    using outputs = type_list<frag_out<PSubj>, scalar_out<StateSubj, ex::lane, life::warp>>;
};
using RowSoftmaxStateUpdate = RowSoftmaxStateUpdateOn<>;
// acc *= exp(m - m') in tensor memory, only when the row maximum grew: reads the accumulator the last P.V commit
// published and publishes the rescaled one to the issuing thread through the mbarrier hand-over that also carries P.
template <class OSubj = sj::Output, class StateSubj = sj::SoftmaxState>
struct RescaleAccumulatorInTmemOn : Obligation<mix3(fnv1a_64_cstr("axp.protocol.softmax.rescale_accumulator_tmem"), OSubj::id, StateSubj::id)> {
    using inputs = type_list<tile_in<sj::in_tmem<OSubj>, ex::warp, life::warp>, scalar_in<StateSubj, ex::lane, life::warp>>;
    using outputs = type_list<tile_out<sj::in_tmem<OSubj>, ex::cta_group1, life::block>>;
};
using RescaleAccumulatorInTmem = RescaleAccumulatorInTmemOn<>;

// Register budget moved from the producer / MMA warpgroup to the math warpgroups.
template <int ProducerRegs, int MathRegs>
struct RoleRegisterBudget : Obligation<mix_u64(fnv1a_64_cstr("axp.protocol.specialize.register_budget"), ProducerRegs * 1024 + MathRegs)> {
    static constexpr int producer_regs = ProducerRegs, math_regs = MathRegs;
};

}  // namespace axp::protocol::sm100
