// GEMM tile recipe on sm100 as an obligation graph.
//
// The reference recipe (include/axp/level3/gemm.hpp:1075-2027) unrolls a
// prologue / steady / drain software pipeline over KTiles with WGMMA obligations
// and ends in shared memory.  The sm100 graph describes the steady-state window
// of a persistent, warp-specialised kernel instead: TMA rings for A and B, one
// tcgen05.mma per 32 bytes of K into a double-buffered TMEM accumulator, and an
// epilogue that reads TMEM, (for scaled recipes) promotes the K-block partial
// with the operand scales into fp32 registers, casts to Recipe::out and stores
// rows to global memory.  KTiles is the window length; the runtime K loop and the
// tile scheduler belong to the kernel.
#pragma once
#include "../graph/flow.hpp"
#include "../kits/intent.hpp"
#include "../kits/sm100/index.hpp"
#include "../naming/subjects.hpp"
#include "../protocol/sm100_contracts.hpp"
#include "epilogue.hpp"
#include "registry.hpp"

namespace axp::level3 {

namespace px = axp::protocol::sm100;

struct gemm_pipe_tag {
    static constexpr auto id = iro::util::fnv1a_64_cstr("axp.level3.gemm.sm100.pipe");
};

template <class Recipe, int BlockM, int BlockN, int BlockK, int Stages, class ASubj, class BSubj, class CSubj, class Cap,
          class MemoryPatternA, class MemoryPatternB, class LoadModeA, class LoadModeB, class Schedule,
          class EpiloguePolicy = epilogue::None, class ScaleASubj = axp::subject::ScaleA, class ScaleBSubj = axp::subject::ScaleB>
struct GemmTileTcgen05Impl {
    using in_a = typename Recipe::in_a;
    using in_b = typename Recipe::in_b;
    using out = typename Recipe::out;
    static_assert(std::is_same_v<typename Recipe::acc, iro::elem::f32>, "tcgen05 accumulates in fp32");
    static_assert(Stages >= 2 && Stages <= 8, "2..8 shared-memory stages");

    // ---- intents -> mechanisms (axp::kit::detail selectors, expert overrides included) ----
    // Both operands are K-major rows of BlockK elements.  The realization stages 128-byte swizzled rows by TMA and runs
    // as a warp-specialised producer / issuer / epilogue pipeline; intents that select anything else have no sm100
    // realization.
    using a_swizzle = axp::kit::detail::select_swizzle_t<MemoryPatternA, in_a, BlockK, Cap, true>;
    using b_swizzle = axp::kit::detail::select_swizzle_t<MemoryPatternB, in_b, BlockK, Cap, false>;
    static_assert(a_swizzle::span_bytes == 128 && b_swizzle::span_bytes == 128,
                  "the sm100 GEMM stages rows of one 128-byte swizzle span: memory_pattern::Optimized with BlockK * bytes == 128");
    static_assert(BlockK * in_a::bytes == 128, "one stage row is one 128-byte swizzle span of K");
    using a_tma = axp::kit::detail::select_tma_t<LoadModeA, Cap, void, ASubj, gemm_pipe_tag>;
    using b_tma = axp::kit::detail::select_tma_t<LoadModeB, Cap, void, BSubj, gemm_pipe_tag>;
    static_assert(axp::kit::detail::is_tma_config_v<a_tma> && axp::kit::detail::is_tma_config_v<b_tma>,
                  "the sm100 GEMM loads its operands by TMA: load_mode::AsyncPrefetch on a TMA target");
    using schedule = axp::kit::detail::select_schedule_t<Schedule, Cap>;
    static_assert(std::is_same_v<schedule, axp::intent::schedule::ProducerConsumer> ||
                      std::is_same_v<schedule, axp::intent::schedule::PersistentPipeline> ||
                      std::is_same_v<schedule, axp::intent::schedule::Pipelined>,
                  "the sm100 GEMM is a persistent producer / consumer pipeline");

    static constexpr int kMmaK = 32 / in_a::bytes;
    // CTA pairs (cta_group::2): a 2*BlockM x BlockN MMA, each CTA loading its own half of A and of B.  Scaled recipes
    // hand the accumulator to the epilogue once per K block; the remote arrive of that hand-over is a relaxed one.
    static constexpr int kCtaGroup = 2;
    static constexpr int kAccStages = 2;
    static constexpr int kTmemCols = kAccStages * BlockN;
    // scaled: two epilogue warpgroups (a thread carries the BlockN / 2 running sums of its row); else four
    static constexpr int kThreads = Recipe::has_scales ? 384 : 640;
    static constexpr int kProducerRegs = Recipe::has_scales ? 40 : 32;
    static constexpr int kEpilogueRegs = Recipe::has_scales ? 232 : 112;
    static constexpr int kABytes = BlockM * BlockK * in_a::bytes;
    static constexpr int kBBytes = BlockN / kCtaGroup * BlockK * in_b::bytes;
    static_assert(Stages * (kABytes + kBBytes) <= Cap::max_smem_bytes, "stage ring exceeds shared memory");

    // wires: A and B travel global -> shared memory; the accumulator wire travels tensor memory -> registers, where the
    // epilogue stages work on it in place; CSubj is the packed result, in registers and then in global memory
    using Acc = axp::subject::Accumulator;
    using mma = px::Tcgen05Mma<BlockM * kCtaGroup, BlockN, kMmaK, in_a, in_b, kCtaGroup, px::OperandSource::shared, px::Major::k, ASubj, BSubj, Acc>;
    using base = iro::util::type_list<
        px::HostMakeTensorMap<ASubj, in_a, 2>, px::HostMakeTensorMap<BSubj, in_b, 2>,
        px::StageRing<ASubj, kABytes, Stages, 2, kCtaGroup>, px::StageRing<BSubj, kBBytes, Stages, 2, kCtaGroup>,
        px::RoleRegisterBudget<kProducerRegs, kEpilogueRegs>, px::TmemAllocate<kTmemCols, kCtaGroup>, px::BoundedBarrierWait, mma,
        px::Tcgen05Commit<kCtaGroup, Acc>, px::TmemToRegisters<32, Acc>>;
    using scale = std::conditional_t<Recipe::has_scales, iro::util::type_list<px::ScalePromoteAccumulator<Recipe, Acc, ScaleASubj, ScaleBSubj>>,
                                     iro::util::type_list<>>;
    using scale_external = std::conditional_t<Recipe::has_scales,
                                              iro::util::concat_t<axp::graph::external_tokens<axp::subject::in_global<ScaleASubj>>,
                                                                  axp::graph::external_tokens<axp::subject::in_global<ScaleBSubj>>>,
                                              iro::util::type_list<>>;
    template <class P, bool = P::enabled>
    struct fused_list {
        using type = iro::util::type_list<>;
        using external = iro::util::type_list<>;
    };
    template <class P, class = void>
    struct fused_one {
        using bias = axp::subject::wire<typename P::bias_tag, 0>;
        using type = px::BiasActivation<bias, typename P::activation, Acc>;
        using external = axp::graph::external_tokens<axp::subject::in_global<bias>>;
    };
    template <class P>
    struct fused_one<P, std::void_t<typename P::up_tag>> {
        // a second tensor map for the up operand, then the gated combine
        using type = px::GatedActivation<axp::subject::wire<typename P::up_tag, 0>, typename P::activation, Acc>;
        using external = iro::util::type_list<>;
    };
    template <class P>
    struct fused_one<P, std::void_t<typename P::c_tag>> {
        using c = axp::subject::wire<typename P::c_tag, 0>;
        using alpha = axp::subject::wire<typename P::alpha_tag, 0>;
        using beta = axp::subject::wire<typename P::beta_tag, 0>;
        using type = px::LinearCombination<c, alpha, beta, Acc>;
        using external = iro::util::concat_t<axp::graph::external_tokens<axp::subject::in_global<c>>,
                                             iro::util::concat_t<axp::graph::external_tokens<alpha>, axp::graph::external_tokens<beta>>>;
    };
    template <class P>
    struct fused_list<P, true> {
        using type = iro::util::type_list<typename fused_one<P>::type>;
        using external = typename fused_one<P>::external;
    };
    using fused = typename fused_list<EpiloguePolicy>::type;
    using tail = iro::util::type_list<px::CastPack<iro::elem::f32, out, typename Recipe::fp8_policy, Acc, CSubj>,
                                      px::StoreRowGlobal<out, CSubj>, px::TmemRelease<kTmemCols, kCtaGroup>>;
    using obligations = iro::util::concat_t<iro::util::concat_t<iro::util::concat_t<base, scale>, fused>, tail>;
    // what the caller hands over: the operands (and scales, bias, C, alpha, beta where the recipe reads them)
    using external_list = iro::util::concat_t<
        iro::util::concat_t<axp::graph::external_tokens<axp::subject::in_global<ASubj>>, axp::graph::external_tokens<axp::subject::in_global<BSubj>>>,
        iro::util::concat_t<scale_external, typename fused_list<EpiloguePolicy>::external>>;

    struct type : iro::compose::Composition<obligations, Cap, kThreads, 232> {
        using recipe = Recipe;
        using external = external_list;
        using carried = iro::util::type_list<>;      // a tile's pipeline starts from nothing: no loop-carried tokens
        static constexpr int block_m = BlockM, block_n = BlockN, block_k = BlockK, stages = Stages;
        static constexpr int cta_group = kCtaGroup, producer_regs = kProducerRegs, epilogue_regs = kEpilogueRegs;
        using a_swizzle = typename GemmTileTcgen05Impl::a_swizzle;
        using b_swizzle = typename GemmTileTcgen05Impl::b_swizzle;
        using a_tma = typename GemmTileTcgen05Impl::a_tma;
        using schedule = typename GemmTileTcgen05Impl::schedule;
        static constexpr int mma_per_stage = BlockK / kMmaK;
        static constexpr bool scaled = Recipe::has_scales;
        static constexpr bool fused_epilogue = EpiloguePolicy::enabled;
    };
    static_assert(axp::kit::sm100::binds_all<obligations>::value, "every obligation needs an sm100 realization");
    using flow = axp::graph::flow<obligations, external_list>;
    static_assert(flow::ports_complete, "a port of the sm100 GEMM graph lacks a token its payload needs");
    static_assert(flow::first_unmet == -1, "an obligation of the sm100 GEMM graph requires a token that nothing before it provides");
};

namespace registry {

template <class Recipe, int BM, int BN, int BK, int Stages, int KTiles, class ASubj, class BSubj, class CSubj, class WgmmaSubj,
          class MPA, class MPB, class LMA, class LMB, class Schedule, class ScaleASubj, class ScaleBSubj, class ATma, class BTma,
          class Cap>
struct resolve_impl<GemmTilePattern<Recipe, BM, BN, BK, Stages, KTiles, ASubj, BSubj, CSubj, WgmmaSubj, MPA, MPB, LMA, LMB,
                                    Schedule, ScaleASubj, ScaleBSubj, ATma, BTma>,
                    Cap, std::enable_if_t<Cap::has_tcgen05>> {
    using type = typename GemmTileTcgen05Impl<Recipe, BM, BN, BK, Stages, ASubj, BSubj, CSubj, Cap, MPA, MPB, LMA, LMB, Schedule, epilogue::None,
                                              ScaleASubj, ScaleBSubj>::type;
};

template <class Recipe, int BM, int BN, int BK, int Stages, int KTiles, class ASubj, class BSubj, class CSubj, class WgmmaSubj,
          class Epi, class MPA, class MPB, class LMA, class LMB, class Schedule, class ScaleASubj, class ScaleBSubj, class ATma,
          class BTma, class Cap>
struct resolve_impl<GemmTileFusedPattern<Recipe, BM, BN, BK, Stages, KTiles, ASubj, BSubj, CSubj, WgmmaSubj, Epi, MPA, MPB, LMA,
                                         LMB, Schedule, ScaleASubj, ScaleBSubj, ATma, BTma>,
                    Cap, std::enable_if_t<Cap::has_tcgen05>> {
    using type = typename GemmTileTcgen05Impl<Recipe, BM, BN, BK, Stages, ASubj, BSubj, CSubj, Cap, MPA, MPB, LMA, LMB, Schedule, Epi, ScaleASubj,
                                              ScaleBSubj>::type;
};

}  // namespace registry
}  // namespace axp::level3
