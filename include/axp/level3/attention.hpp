// Attention tile recipe on sm100 as an obligation graph.
//
// Reference dataflow per (Q tile, KV tile) step (include/axp/level3/recipes/
// attention/process.hpp:1766-1864): QK -> mask -> softmax(+state) -> combine ->
// rescale accumulator -> scale weights -> cast P -> PV -> add.  The sm100 graph
// keeps the same steps with the softmax state per query row, S and O in tensor
// memory, P either overwriting its S region (16-bit: the tensor-memory A operand of
// the PV MMA) or passing through shared memory (8-bit), V the MN-major B operand,
// and the accumulator rescale applied in place only when a row maximum grew.  The reference restricts attention inputs to f16/bf16
// (include/axp/level3/attention.hpp:95-96); the E4M3 branch is an sm100 addition.
#pragma once
#include "../graph/flow.hpp"
#include "../kits/intent.hpp"
#include "../kits/sm100/index.hpp"
#include "../protocol/sm100_contracts.hpp"
#include "../state.hpp"
#include "registry.hpp"

namespace axp::level3 {

namespace px = axp::protocol::sm100;

struct attention_pipe_tag {
    static constexpr auto id = iro::util::fnv1a_64_cstr("axp.level3.attention.sm100.pipe");
};
struct attention_p_tag {
    static constexpr auto id = iro::util::fnv1a_64_cstr("axp.level3.attention.sm100.p");
};

template <class Recipe, int TileQ, int TileK, int TileV, int HeadDim, int Stages, class QSubj, class KSubj, class VSubj,
          class MemoryPatternQ, class MemoryPatternK, class MemoryPatternV, class LoadModeQ, class LoadModeK, class LoadModeV,
          class Schedule, class TileSkip, class Cap>
struct AttentionTileTcgen05Impl {
    using in = typename Recipe::in_a;
    using out = typename Recipe::out;
    static_assert(TileK == TileV, "K and V tiles cover the same keys (reference attention.hpp:808)");
    static_assert(TileQ == 128 && TileK == 128 && HeadDim == 128, "realised tile: 128 queries x 128 keys x 128 head dim");
    static_assert(Stages >= 2 && Stages <= 4, "2..4 K/V stages");

    // ---- intents -> mechanisms ----
    // Q and K rows are HeadDim elements (K-major operands of Q.K^T), V rows are its MN-major B operand: all are staged
    // as 128-byte swizzle spans by TMA.
    using q_swizzle = axp::kit::detail::select_swizzle_t<MemoryPatternQ, in, HeadDim, Cap, true>;
    using k_swizzle = axp::kit::detail::select_swizzle_t<MemoryPatternK, in, HeadDim, Cap, true>;
    using v_swizzle = axp::kit::detail::select_swizzle_t<MemoryPatternV, in, HeadDim, Cap, false>;
    static_assert(q_swizzle::span_bytes == 128 && k_swizzle::span_bytes == 128 && v_swizzle::span_bytes == 128,
                  "the sm100 attention stages 128-byte swizzle spans: memory_pattern::Optimized");
    using q_tma = axp::kit::detail::select_tma_t<LoadModeQ, Cap, void, QSubj, attention_pipe_tag>;
    using k_tma = axp::kit::detail::select_tma_t<LoadModeK, Cap, void, KSubj, attention_pipe_tag>;
    using v_tma = axp::kit::detail::select_tma_t<LoadModeV, Cap, void, VSubj, attention_pipe_tag>;
    static_assert(axp::kit::detail::is_tma_config_v<q_tma> && axp::kit::detail::is_tma_config_v<k_tma> && axp::kit::detail::is_tma_config_v<v_tma>,
                  "the sm100 attention loads Q, K and V by TMA: load_mode::AsyncPrefetch on a TMA target");
    using schedule = axp::kit::detail::select_schedule_t<Schedule, Cap>;

    static constexpr int kQTilesPerCta = 2;
    static constexpr int kMmaK = 32 / in::bytes;
    // 16-bit operands: the 128 keys of the intent tile are taken in two steps of 64 (two 64-column S buffers per Q tile,
    // so that the next Q.K^T is in flight while the softmax runs) and P overwrites its S region in tensor memory.
    // 8-bit operands: steps of 128 keys, P goes to the P.V MMA through shared memory (two tiles per Q tile).
    static constexpr bool kPThroughSmem = in::bytes == 1;
    static constexpr int kKvStep = in::bytes == 2 ? 64 : 128;
    static constexpr int kQTileBytes = TileQ * HeadDim * in::bytes;
    static constexpr int kKvTileBytes = kKvStep * HeadDim * in::bytes;
    static constexpr int kTmemCols = 512;   // S0 S1 O0 O1, 128 fp32 columns each
    static constexpr int kThreads = 384;    // two softmax warpgroups (one per Q tile), TMA producer warp, two issuing warps
    static constexpr int kProducerRegs = 56, kSoftmaxRegs = 224;
    static constexpr int kIssuers = 2;
    static constexpr bool causal = std::is_same_v<TileSkip, axp::intent::tile_skip::Causal>;

    // wires: S = scores (tensor memory -> registers), P = weights (registers -> tensor or shared memory), O = the output
    // accumulator in tensor memory and, after the last step, the packed result in registers and global memory; the per-row
    // (m, l) state lives in registers of the row's thread
    using S = axp::subject::AttentionS;
    using P = axp::subject::AttentionP;
    using O = axp::subject::Output;
    using State = axp::subject::SoftmaxState;
    using qk = px::Tcgen05Mma<TileQ, kKvStep, kMmaK, in, in, 1, px::OperandSource::shared, px::Major::k, QSubj, KSubj, S>;
    using pv = px::Tcgen05Mma<TileQ, HeadDim, kMmaK, in, in, 1, (kPThroughSmem ? px::OperandSource::shared : px::OperandSource::tmem),
                              px::Major::mn, P, VSubj, O>;
    using p_route = std::conditional_t<kPThroughSmem, px::RegistersToSharedOperand<kQTileBytes, 2 * kQTilesPerCta, P>, px::RegistersToTmem<32, P>>;
    // one step of the KV loop, then the epilogue of the Q tile
    using obligations = iro::util::type_list<
        px::HostMakeTensorMap<QSubj, in, 3>, px::HostMakeTensorMap<KSubj, in, 3>, px::HostMakeTensorMap<VSubj, in, 3>,
        px::StageRing<QSubj, kQTileBytes, kQTilesPerCta, 3>, px::StageRing<KSubj, kKvTileBytes, Stages, 3>,
        px::StageRing<VSubj, kKvTileBytes, Stages, 3>, px::RoleRegisterBudget<kProducerRegs, kSoftmaxRegs>, px::TmemAllocate<kTmemCols, 1>,
        px::BoundedBarrierWait, qk, px::Tcgen05Commit<1, S>, px::TmemToRegisters<32, S>, px::CausalMaskPredicate<TileQ, kKvStep, S>,
        px::RowSoftmaxStateUpdateOn<S, P, State>, px::RescaleAccumulatorInTmemOn<O, State>, px::CastWeights<in, typename Recipe::fp8_policy, P>,
        p_route, pv, px::Tcgen05Commit<1, O>, px::TmemToRegisters<32, O>,
        px::CastPack<iro::elem::f32, out, typename Recipe::fp8_policy, O, O>, px::StoreRowGlobal<out, O>,
        px::TmemRelease<kTmemCols, 1>>;
    using external_list = iro::util::concat_t<axp::graph::external_tokens<axp::subject::in_global<QSubj>>,
                                              iro::util::concat_t<axp::graph::external_tokens<axp::subject::in_global<KSubj>>,
                                                                  axp::graph::external_tokens<axp::subject::in_global<VSubj>>>>;
    // carried from the previous step of the KV loop: the accumulator that the last P.V commit published (the rescale
    // reads it) and the rows' (m, l); the list must provide both again
    using carried_list = iro::util::type_list<iro::token::visible_at<axp::subject::in_tmem<O>, iro::scope::block>,
                                              iro::token::alive<axp::subject::in_tmem<O>, iro::token::lifetime::block>,
                                              iro::token::alive<State, iro::token::lifetime::warp>>;

    struct type : iro::compose::Composition<obligations, Cap, kThreads, kSoftmaxRegs> {
        using recipe = Recipe;
        using state = axp::state::SoftmaxStateF32;
        using external = external_list;
        using carried = carried_list;
        static constexpr int tile_q = TileQ, tile_k = TileK, head_dim = HeadDim, stages = Stages;
        static constexpr int kv_step = kKvStep, q_tiles = kQTilesPerCta, issuers = kIssuers;
        static constexpr int producer_regs = kProducerRegs, softmax_regs = kSoftmaxRegs;
        static constexpr bool p_through_smem = kPThroughSmem;
        static constexpr bool is_causal = causal;
        using q_swizzle = typename AttentionTileTcgen05Impl::q_swizzle;
        using schedule = typename AttentionTileTcgen05Impl::schedule;
    };
    static_assert(axp::kit::sm100::binds_all<obligations>::value, "every obligation needs an sm100 realization");
    using flow = axp::graph::flow<obligations, external_list, carried_list>;
    static_assert(flow::ports_complete, "a port of the sm100 attention graph lacks a token its payload needs");
    static_assert(flow::first_unmet == -1, "an obligation of the sm100 attention graph requires a token that nothing before it provides");
    static_assert(flow::carried_closed, "the KV step does not provide again what it takes from the previous step");
};

namespace registry {

template <class Recipe, int TQ, int TK, int TV, int HD, int Stages, int SlotIdx, class QSubj, class KSubj, class VSubj,
          class AccSubj, class OldS, class OutS, class MPQ, class MPK, class MPV, class LMQ, class LMK, class LMV, class Schedule,
          class TileSkip, class QTma, class KTma, class VTma, class Cap>
struct resolve_impl<AttentionTilePattern<Recipe, TQ, TK, TV, HD, Stages, SlotIdx, QSubj, KSubj, VSubj, AccSubj, OldS, OutS, MPQ,
                                         MPK, MPV, LMQ, LMK, LMV, Schedule, TileSkip, QTma, KTma, VTma>,
                    Cap, std::enable_if_t<Cap::has_tcgen05>> {
    using type = typename AttentionTileTcgen05Impl<Recipe, TQ, TK, TV, HD, Stages, QSubj, KSubj, VSubj, MPQ, MPK, MPV, LMQ, LMK, LMV, Schedule,
                                                   TileSkip, Cap>::type;
};

}  // namespace registry
}  // namespace axp::level3
