// Compile-time checks of the sm100 rows: every manifest row resolves through
// L4 preset -> L4->L3 lowering -> level3::registry::Select<Pattern, cap::sm100> ->
// axp::l4::resolve, with the declared graph hash, realization key and bind key, and
// every obligation of the selected graphs binds to an sm100 realization.
// Mirrors the reference's static_assert suites (tests/compile/ax_asserts.cu:193-204
// for capability flags, tests/compile/ax_asserts_primitives.cu:708-739 for
// resolution) and its per-row generated TUs (tools/ax_manifest_tool.cpp:1328-1371).
#define AXP_LIBRARY_BUILD
#define AXP_ENABLE_SM100
#ifndef AXP_TARGET_SM
#define AXP_TARGET_SM 1000
#endif
#include <axp/l4/resolve.hpp>

#include "../../iro-cuda-ax_b200/csrc/kernel_config.hpp"   // the configuration the kernel translation units are checked against

namespace {

using iro::util::fnv1a_64_cstr;
using Cap = iro::cap::sm100;
using Prof = axp::l4::profile::proof_full;
namespace preset = axp::l4::preset;
namespace px = axp::protocol::sm100;

// ---- substrate ---------------------------------------------------------------
static_assert(fnv1a_64_cstr("") == 14695981039346656037ULL);
static_assert(fnv1a_64_cstr("a") == 0xaf63dc4c8601ec8cULL);
static_assert(std::is_same_v<axp::target_cap, Cap>);
static_assert(Cap::has_tma && Cap::has_tcgen05 && !Cap::has_wgmma);
static_assert(Cap::max_smem_bytes == 227 * 1024 && Cap::tmem_columns == 512);
static_assert(iro::elem::e4m3::bytes == 1 && iro::elem::bf16::bytes == 2 && iro::elem::f32::bytes == 4);
static_assert(axp::recipe::E4M3BlockScaledAccF32OutBF16::has_scales && !axp::recipe::BF16AccF32Fast::has_scales);
static_assert(axp::recipe::E4M3BlockScaledAccF32OutBF16::scale_vec_a == 1 &&
              axp::recipe::E4M3BlockScaledAccF32OutBF16::scale_vec_b == 128);

// ---- tcgen05 shapes ------------------------------------------------------------
static_assert(px::is_tcgen05_shape_v<128, 256, 32, 1, 1>);     // fp8, one CTA
static_assert(px::is_tcgen05_shape_v<128, 256, 16, 2, 1>);     // bf16
static_assert(px::is_tcgen05_shape_v<256, 256, 16, 2, 2>);     // CTA pair
static_assert(!px::is_tcgen05_shape_v<128, 256, 16, 1, 1>);    // K must span 32 bytes
static_assert(!px::is_tcgen05_shape_v<128, 264, 16, 2, 1>);    // N <= 256
static_assert(!px::is_tcgen05_shape_v<192, 128, 16, 2, 1>);    // M in {64,128} for one CTA

template <class Preset>
using Graph = axp::level3::registry::Select<axp::l4::lowering::to_l3_pattern_t<Preset>, Cap>;

// ---- one block per manifest row -------------------------------------------------
template <class Preset, iro::util::u64 Hash, iro::util::u64 Key>
constexpr bool row_resolves() {
    using G = Graph<Preset>;
    using R = axp::l4::resolve<G, Cap, Prof>;
    static_assert(axp::graph::verify<G>());
    static_assert(R::graph_hash == Hash, "declared graph hash");
    static_assert(R::realization_key == Key, "realization key = fnv1a_64(manifest realization_key)");
    static_assert(std::is_same_v<typename R::l4_pattern, Preset>);
    static_assert(std::is_same_v<typename R::type, G>, "Selected == Graph");
    static_assert(R::bind_key == axp::l4::bind_key_v<Hash, Cap, Prof, Key>);
    static_assert(axp::l4::supports<G, Cap, Prof>::value);
    static_assert(!axp::l4::supports<G, Cap, axp::l4::profile::dev_fast>::value, "only proof_full rows are declared");
    return true;
}

static_assert(row_resolves<preset::GemmFp8BlockScaled128x256x128, fnv1a_64_cstr("axp.sm100.gemm_fp8_blockscaled_128x256x128"),
                           fnv1a_64_cstr("preset.gemm.fp8bs.128x256x128")>());
static_assert(row_resolves<preset::GemmBf16_128x256x64, fnv1a_64_cstr("axp.sm100.gemm_bf16_128x256x64"),
                           fnv1a_64_cstr("preset.gemm.bf16.128x256x64")>());
static_assert(row_resolves<preset::Attention128x128x128CausalBf16, fnv1a_64_cstr("axp.sm100.attention_bf16_128x128x128_causal"),
                           fnv1a_64_cstr("preset.attention.bf16.128x128x128.causal")>());
static_assert(row_resolves<preset::Attention128x128x128CausalFp8Gqa, fnv1a_64_cstr("axp.sm100.attention_fp8_gqa_128x128x128_causal"),
                           fnv1a_64_cstr("preset.attention.fp8.gqa.128x128x128.causal")>());

static_assert(row_resolves<preset::GemmBf16_128x256x64BiasSiLU, fnv1a_64_cstr("axp.sm100.gemm_bf16_128x256x64_bias_silu"),
                           fnv1a_64_cstr("preset.gemm_fused.bf16.128x256x64.bias_silu")>());

static_assert(row_resolves<preset::GemmBf16_128x256x64SwiGLU, fnv1a_64_cstr("axp.sm100.gemm_bf16_128x256x64_swiglu"),
                           fnv1a_64_cstr("preset.gemm_fused.bf16.128x256x64.swiglu")>());

static_assert(row_resolves<preset::GemmBf16_128x256x64LinComb, fnv1a_64_cstr("axp.sm100.gemm_bf16_128x256x64_lincomb"),
                           fnv1a_64_cstr("preset.gemm_fused.bf16.128x256x64.lincomb")>());

// ---- graph contents ---------------------------------------------------------------
using GFp8 = Graph<preset::GemmFp8BlockScaled128x256x128>;
using GBf16 = Graph<preset::GemmBf16_128x256x64>;
using GAttn = Graph<preset::Attention128x128x128CausalBf16>;
using GAttn8 = Graph<preset::Attention128x128x128CausalFp8Gqa>;
static_assert(GFp8::scaled && !GBf16::scaled);
static_assert(GFp8::smem_bytes == 6 * (128 * 128 + 128 * 128) && GFp8::tmem_cols == 512 && GFp8::mma_per_stage == 4);
static_assert(GBf16::smem_bytes == 6 * (128 * 128 + 128 * 128) && GBf16::mma_per_stage == 4 && GBf16::threads == 640);

// ---- the graphs describe the kernels the default dispatch launches ---------------------
namespace cfg = axp_shim::cfg;
template <class G>
constexpr bool gemm_graph_matches(const cfg::Gemm& k) {
    return G::block_m == k.tile_m && G::block_n == k.tile_n && G::block_k == k.tile_k && G::cta_group == k.cta_group && G::stages == k.stages &&
           G::smem_bytes == k.stages * k.stage_bytes && G::smem_bytes + 1024 == k.dyn_smem && G::tmem_cols == k.tmem_cols &&
           G::threads == k.threads && G::producer_regs == k.producer_regs && G::epilogue_regs == k.epilogue_regs;
}
template <class G>
constexpr bool attention_graph_matches(const cfg::Attn& k) {
    return G::tile_q == k.tile_q && G::kv_step == k.kv_tile && G::head_dim == k.head_dim && G::q_tiles == k.q_tiles && G::stages == k.kv_stages &&
           G::smem_bytes + 1024 == k.dyn_smem && G::tmem_cols == k.tmem_cols && G::threads == k.threads && G::producer_regs == k.producer_regs &&
           G::softmax_regs == k.softmax_regs && G::issuers == k.issuers && G::p_through_smem == k.p_through_smem;
}
static_assert(gemm_graph_matches<GFp8>(cfg::kGemmFp8), "level-3 graph of the FP8 GEMM row and the launched kernel differ");
static_assert(gemm_graph_matches<GBf16>(cfg::kGemmBf16), "level-3 graph of the bf16 GEMM row and the launched kernel differ");
static_assert(gemm_graph_matches<Graph<preset::GemmBf16_128x256x64BiasSiLU>>(cfg::kGemmBf16));
static_assert(attention_graph_matches<GAttn>(cfg::kAttnBf16), "level-3 graph of the bf16 attention row and the launched kernel differ");
static_assert(attention_graph_matches<GAttn8>(cfg::kAttnFp8), "level-3 graph of the E4M3 attention row and the launched kernel differ");

// ---- intent selectors (include/axp/kits/intent.hpp) -----------------------------------------
namespace kd = axp::kit::detail;
namespace mp = axp::intent::memory_pattern;
namespace lm = axp::intent::load_mode;
static_assert(std::is_same_v<kd::select_swizzle_t<mp::Optimized, iro::elem::e4m3, 128, Cap, true>, axp::swizzle::B128>);
static_assert(std::is_same_v<kd::select_swizzle_t<mp::Optimized, iro::elem::bf16, 64, Cap, false>, axp::swizzle::B128>);
static_assert(std::is_same_v<kd::select_swizzle_t<mp::Optimized, iro::elem::bf16, 32, Cap, true>, axp::swizzle::B64>);
static_assert(std::is_same_v<kd::select_swizzle_t<mp::Optimized, iro::elem::e4m3, 32, Cap, true>, axp::swizzle::B32>);
static_assert(std::is_same_v<kd::select_swizzle_t<mp::Optimized, iro::elem::e4m3, 16, Cap, true>, axp::swizzle::None>);
static_assert(std::is_same_v<kd::select_swizzle_t<mp::None, iro::elem::bf16, 64, Cap, true>, axp::swizzle::None>);
static_assert(kd::is_tma_config_v<kd::select_tma_t<lm::AsyncPrefetch, Cap, void, preset::GemmA, axp::level3::gemm_pipe_tag>>);
static_assert(std::is_same_v<kd::select_tma_t<lm::Streaming, Cap, void, preset::GemmA, axp::level3::gemm_pipe_tag>, kd::streaming_tag>);
static_assert(std::is_same_v<kd::select_schedule_t<axp::intent::schedule::ProducerConsumer, Cap>, axp::intent::schedule::ProducerConsumer>);
static_assert(std::is_same_v<GFp8::a_swizzle, axp::swizzle::B128> && std::is_same_v<GAttn::q_swizzle, axp::swizzle::B128>);
static_assert(axp::swizzle::B128::tensor_map_swizzle == 3 && axp::swizzle::B128::descriptor_code == 2);
static_assert(iro::util::contains<px::ScalePromoteAccumulator<axp::recipe::E4M3BlockScaledAccF32OutBF16>, GFp8::obligations>::value);
static_assert(!iro::util::contains<px::ScalePromoteAccumulator<axp::recipe::E4M3BlockScaledAccF32OutBF16>, GBf16::obligations>::value);
using GFused = Graph<preset::GemmBf16_128x256x64BiasSiLU>;
static_assert(GFused::fused_epilogue && !GBf16::fused_epilogue && GFused::id != GBf16::id);
static_assert(iro::util::contains<px::BiasActivation<preset::GemmBiasSiLU, axp::level3::epilogue::act::SiLU>, GFused::obligations>::value);
using GLin = Graph<preset::GemmBf16_128x256x64LinComb>;
static_assert(iro::util::contains<px::LinearCombination<preset::GemmLinCombC, axp::subject::wire<preset::GemmLinCombAlphaTag, 0>,
                                                         axp::subject::wire<preset::GemmLinCombBetaTag, 0>>, GLin::obligations>::value);
static_assert(GLin::id != GFused::id);
using GSwi = Graph<preset::GemmBf16_128x256x64SwiGLU>;
static_assert(iro::util::contains<px::GatedActivation<preset::GemmUpOperand, axp::level3::epilogue::act::SiLU>, GSwi::obligations>::value);
static_assert(GSwi::id != GFused::id);
static_assert(GAttn::is_causal && GAttn::tmem_cols == 512 && GAttn::smem_bytes == 2 * 32768 + 2 * 4 * 16384);
static_assert(GAttn8::smem_bytes == (2 + 4 + 2 * 3) * 16384);      // Q tiles, P tiles, K / V stages
static_assert(GFp8::id != GBf16::id && GAttn::id != GAttn8::id, "distinct obligation lists hash differently");

// ---- kit binding --------------------------------------------------------------------
using MmaFp8 = px::Tcgen05Mma<128, 256, 32, iro::elem::e4m3, iro::elem::e4m3, 1>;
static_assert(axp::kit::sm100::bind<MmaFp8>::found);
static_assert(std::is_same_v<axp::kit::sm100::bind<MmaFp8>::realization::obligation, MmaFp8>);
static_assert(axp::kit::sm100::bind<MmaFp8>::realization::impl_id == fnv1a_64_cstr("axp.realize.sm100.compute.tcgen05_mma_ss"));
// the realization id mixes obligation and implementation (reference include/iro_cuda_ax_core.hpp:3290-3300)
static_assert(axp::kit::sm100::bind<MmaFp8>::realization::id ==
              iro::util::mix_u64(fnv1a_64_cstr("iro.contract.Realization"),
                                 iro::util::mix_u64(MmaFp8::id, fnv1a_64_cstr("axp.realize.sm100.compute.tcgen05_mma_ss"))));
// every leaf of every bound realization carries an execute member (the kernels call these)
static_assert(axp::kit::sm100::binds_all<GFp8::obligations>::value && axp::kit::sm100::binds_all<GAttn8::obligations>::value);
static_assert(axp::kit::sm100::detail::has_execute<axp::realize::sm100::ScalePromoteFma>::value &&
              axp::kit::sm100::detail::has_execute<axp::realize::sm100::TmemLoadWait>::value &&
              axp::kit::sm100::detail::has_execute<axp::realize::sm100::HostTensorMapEncoder>::value &&
              axp::kit::sm100::detail::has_execute<axp::realize::sm100::CausalMaskPred>::value);
// calling a realization the way the reference's example does (examples/sm89_ax_div_example.cu:20-41): bind, take the leaf, execute
using PromoteBound = axp::kit::sm100::bind<px::ScalePromoteAccumulator<axp::recipe::E4M3BlockScaledAccF32OutBF16>>;
static_assert(std::is_same_v<iro::util::front_t<PromoteBound::realization::leaves>, axp::realize::sm100::ScalePromoteFma>);
struct NoExecuteProbe {};
static_assert(!axp::kit::sm100::detail::has_execute<NoExecuteProbe>::value);
static_assert(iro::util::contains<axp::realize::sm100::Tcgen05Mma<1, false>, axp::kit::sm100::bind<MmaFp8>::realization::leaves>::value);
static_assert(axp::kit::sm100::bind<px::BoundedBarrierWait>::found);

// ---- tokens, ports and contract flow ---------------------------------------------------
// (reference: contract_tokens_complete pins Tcgen05Mma and the tensor-memory moves,
// tests/compile/ax_asserts_primitives.cu:146-155,571-576; rules in include/axp/protocol/audit/tokens.hpp:35-80)
namespace flowtest {
namespace sj = axp::subject;
namespace tk = iro::token;
namespace audit = axp::protocol::audit;
using iro::util::type_list;
using Acc = sj::Accumulator;
using e4 = iro::elem::e4m3;
using b16 = iro::elem::bf16;

// every obligation kind of the two graphs names complete token lists on its ports
using MmaPair = px::Tcgen05Mma<256, 256, 32, e4, e4, 2, px::OperandSource::shared, px::Major::k, sj::MatrixA, sj::MatrixB, Acc>;
using MmaOne = px::Tcgen05Mma<128, 256, 32, e4, e4, 1, px::OperandSource::shared, px::Major::k, sj::MatrixA, sj::MatrixB, Acc>;
using MmaTs = px::Tcgen05Mma<128, 128, 16, b16, b16, 1, px::OperandSource::tmem, px::Major::mn, sj::AttentionP, sj::AttentionV, sj::Output>;
static_assert(audit::contract_tokens_complete<MmaPair>() && audit::contract_tokens_complete<MmaOne>() && audit::contract_tokens_complete<MmaTs>());
static_assert(audit::contract_tokens_complete<px::Tcgen05Commit<2, Acc>>() && audit::contract_tokens_complete<px::TmemToRegisters<32, Acc>>() &&
              audit::contract_tokens_complete<px::RegistersToTmem<32, sj::AttentionP>>() &&
              audit::contract_tokens_complete<px::RegistersToSharedOperand<16384, 4, sj::AttentionP>>());
static_assert(audit::contract_tokens_complete<px::HostMakeTensorMap<sj::MatrixA, e4, 2>>() &&
              audit::contract_tokens_complete<px::StageRing<sj::MatrixA, 16384, 6, 2, 2>>() && audit::contract_tokens_complete<px::TmemAllocate<512, 2>>() &&
              audit::contract_tokens_complete<px::TmemRelease<512, 2>>() && audit::contract_tokens_complete<px::BoundedBarrierWait>());
static_assert(audit::contract_tokens_complete<px::ScalePromoteAccumulator<axp::recipe::E4M3BlockScaledAccF32OutBF16>>() &&
              audit::contract_tokens_complete<px::CastPack<iro::elem::f32, b16, iro::recipe::fp8_native>>() &&
              audit::contract_tokens_complete<px::StoreRowGlobal<b16>>() && audit::contract_tokens_complete<px::CausalMaskPredicate<128, 64>>() &&
              audit::contract_tokens_complete<px::RowSoftmaxStateUpdate>() && audit::contract_tokens_complete<px::RescaleAccumulatorInTmem>() &&
              audit::contract_tokens_complete<px::CastWeights<b16, iro::recipe::fp8_native>>());
// the operands of a pair MMA must be published at cluster scope, its result is visible to the issuing lane only
using PairA = iro::util::front_t<MmaPair::inputs>;
static_assert(PairA::is_input && std::is_same_v<PairA::subject, sj::in_shared<sj::MatrixA>> && std::is_same_v<PairA::exec_group, iro::exec::cta_group2>);
static_assert(iro::verify::has_token_kind_subject<PairA::required, tk::kind_sync_at, sj::in_shared<sj::MatrixA>>());
static_assert(std::is_same_v<iro::util::front_t<iro::util::front_t<MmaPair::outputs>::provided>, tk::visible_at<sj::in_tmem<Acc>, iro::scope::lane>>);
// the audit rejects incomplete ports: a tile without liveness; a block-wide output without its synchronisation
using NoAlive = iro::contract::InputPort<iro::contract::Tile<iro::contract::space::shared>, sj::in_shared<sj::MatrixA>, iro::exec::warp,
                                         type_list<tk::visible_at<sj::in_shared<sj::MatrixA>, iro::scope::warp>>>;
using NoSync = iro::contract::OutputPort<iro::contract::Tile<iro::contract::space::tmem>, sj::in_tmem<Acc>, iro::exec::cta_group1,
                                         type_list<tk::visible_at<sj::in_tmem<Acc>, iro::scope::block>, tk::alive<sj::in_tmem<Acc>, tk::lifetime::block>>>;
using LaneOut = iro::contract::OutputPort<iro::contract::Tile<iro::contract::space::tmem>, sj::in_tmem<Acc>, iro::exec::lane,
                                          type_list<tk::visible_at<sj::in_tmem<Acc>, iro::scope::lane>, tk::alive<sj::in_tmem<Acc>, tk::lifetime::block>>>;
static_assert(!audit::port_tokens_complete<NoAlive>() && !audit::port_tokens_complete<NoSync>() && audit::port_tokens_complete<LaneOut>());
// satisfies: same kind and subject at a scope at least as wide
static_assert(iro::verify::satisfies_v<type_list<tk::visible_at<Acc, iro::scope::block>>, tk::visible_at<Acc, iro::scope::warp>>);
static_assert(!iro::verify::satisfies_v<type_list<tk::visible_at<Acc, iro::scope::lane>>, tk::visible_at<Acc, iro::scope::warp>>);
static_assert(!iro::verify::satisfies_v<type_list<tk::visible_at<sj::Output, iro::scope::block>>, tk::visible_at<Acc, iro::scope::warp>>);

// flow over hand-made lists: the GEMM chain closes; taking a link out names the obligation that is left without its token
using Ext = iro::util::concat_t<axp::graph::external_tokens<sj::in_global<sj::MatrixA>>, axp::graph::external_tokens<sj::in_global<sj::MatrixB>>>;
using Good = type_list<px::HostMakeTensorMap<sj::MatrixA, e4, 2>, px::HostMakeTensorMap<sj::MatrixB, e4, 2>, px::StageRing<sj::MatrixA, 16384, 6, 2, 2>,
                       px::StageRing<sj::MatrixB, 16384, 6, 2, 2>, px::TmemAllocate<512, 2>, MmaPair, px::Tcgen05Commit<2, Acc>,
                       px::TmemToRegisters<32, Acc>, px::CastPack<iro::elem::f32, b16, iro::recipe::fp8_native, Acc, sj::MatrixC>,
                       px::StoreRowGlobal<b16, sj::MatrixC>, px::TmemRelease<512, 2>>;
static_assert(axp::graph::flow<Good, Ext>::closed);
// no tcgen05.commit between the MMA and the tensor-memory read: the read (index 6) has nothing that published the accumulator
using NoCommit = type_list<px::HostMakeTensorMap<sj::MatrixA, e4, 2>, px::HostMakeTensorMap<sj::MatrixB, e4, 2>, px::StageRing<sj::MatrixA, 16384, 6, 2, 2>,
                           px::StageRing<sj::MatrixB, 16384, 6, 2, 2>, px::TmemAllocate<512, 2>, MmaPair, px::TmemToRegisters<32, Acc>>;
static_assert(axp::graph::flow<NoCommit, Ext>::first_unmet == 6);
// B never staged: the MMA (index 4) lacks its operand
using NoRingB = type_list<px::HostMakeTensorMap<sj::MatrixA, e4, 2>, px::HostMakeTensorMap<sj::MatrixB, e4, 2>, px::StageRing<sj::MatrixA, 16384, 6, 2, 2>,
                          px::TmemAllocate<512, 2>, MmaPair>;
static_assert(axp::graph::flow<NoRingB, Ext>::first_unmet == 4);
// rings filled per CTA feeding a pair MMA: published at block scope, required at cluster scope
using BlockRings = type_list<px::HostMakeTensorMap<sj::MatrixA, e4, 2>, px::HostMakeTensorMap<sj::MatrixB, e4, 2>, px::StageRing<sj::MatrixA, 16384, 6, 2, 1>,
                             px::StageRing<sj::MatrixB, 16384, 6, 2, 1>, px::TmemAllocate<512, 2>, MmaPair>;
static_assert(axp::graph::flow<BlockRings, Ext>::first_unmet == 5);
// no tensor map: the ring (index 0) cannot issue its copies; no tensor-memory allocation: the MMA cannot name its accumulator
static_assert(axp::graph::flow<type_list<px::StageRing<sj::MatrixA, 16384, 6, 2, 2>>, Ext>::first_unmet == 0);
using NoAlloc = type_list<px::HostMakeTensorMap<sj::MatrixA, e4, 2>, px::HostMakeTensorMap<sj::MatrixB, e4, 2>, px::StageRing<sj::MatrixA, 16384, 6, 2, 2>,
                          px::StageRing<sj::MatrixB, 16384, 6, 2, 2>, MmaPair>;
static_assert(axp::graph::flow<NoAlloc, Ext>::first_unmet == 4);
// an operand nobody handed to the kernel
static_assert(axp::graph::flow<Good, axp::graph::external_tokens<sj::in_global<sj::MatrixA>>>::first_unmet == 1);

// loop-carried tokens: a KV step that takes the published accumulator from the previous step must publish it again
using O = sj::Output;
using CarriedO = type_list<tk::visible_at<sj::in_tmem<O>, iro::scope::block>, tk::alive<sj::in_tmem<O>, tk::lifetime::block>>;
using StepOpen = type_list<px::TmemAllocate<512, 1>, px::RescaleAccumulatorInTmemOn<O, sj::SoftmaxState>>;
using CarriedState = iro::util::concat_t<CarriedO, type_list<tk::alive<sj::SoftmaxState, tk::lifetime::warp>>>;
static_assert(axp::graph::flow<StepOpen, type_list<>, CarriedState>::first_unmet == -1);
static_assert(!axp::graph::flow<StepOpen, type_list<>, CarriedState>::carried_closed, "the state is taken and never provided again");

// the shipped graphs: closed, and every row's graph passes verify (which includes the flow)
template <class Preset>
constexpr bool graph_flow_closed() {
    using G = Graph<Preset>;
    using F = axp::graph::flow<typename G::obligations, typename G::external, typename G::carried>;
    return F::ports_complete && F::first_unmet == -1 && F::carried_closed && axp::graph::flow_closed<G>();
}
static_assert(graph_flow_closed<preset::GemmFp8BlockScaled128x256x128>() && graph_flow_closed<preset::GemmBf16_128x256x64>() &&
              graph_flow_closed<preset::GemmBf16_128x256x64BiasSiLU>() && graph_flow_closed<preset::GemmBf16_128x256x64SwiGLU>() &&
              graph_flow_closed<preset::GemmBf16_128x256x64LinComb>() && graph_flow_closed<preset::Attention128x128x128CausalBf16>() &&
              graph_flow_closed<preset::Attention128x128x128CausalFp8Gqa>());
// the attention step carries the accumulator and the row state; the GEMM carries nothing
static_assert(Graph<preset::Attention128x128x128CausalBf16>::carried::size == 3 && Graph<preset::GemmBf16_128x256x64>::carried::size == 0);
// the E4M3 attention routes P through shared memory, the bf16 one through tensor memory: the P.V MMA's A port follows
using AttnF8 = Graph<preset::Attention128x128x128CausalFp8Gqa>;
using AttnBf = Graph<preset::Attention128x128x128CausalBf16>;
static_assert(iro::util::contains<px::RegistersToSharedOperand<16384, 4, sj::AttentionP>, AttnF8::obligations>::value);
static_assert(iro::util::contains<px::RegistersToTmem<32, sj::AttentionP>, AttnBf::obligations>::value);
}  // namespace flowtest

// ---- not realised on sm100 ----------------------------------------------------------
using F16Gemm = axp::level3::registry::GemmTilePattern<axp::recipe::F16AccF32Fast, 128, 256, 48, 4, 5, preset::GemmA, preset::GemmB,
                                                       preset::GemmC, preset::GemmAcc, axp::intent::memory_pattern::Optimized,
                                                       axp::intent::memory_pattern::Optimized, axp::intent::load_mode::AsyncPrefetch,
                                                       axp::intent::load_mode::AsyncPrefetch, axp::intent::schedule::Pipelined>;
static_assert(!axp::level3::registry::supports<F16Gemm, iro::cap::sm90>::value, "this tree has no sm90 lane");

}  // namespace

// device instantiation of a few leaves, so that the PTX of the atoms is assembled for sm_100a
__global__ void axp_sm100_leaf_instantiation(unsigned* out) {
    namespace rz = axp::realize::sm100;
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        rz::BarrierInit::execute(&bar, 1);
        rz::BarrierInitFence::execute();
        rz::BarrierArrive::execute(&bar);
        out[0] = rz::BarrierTryWait::execute(&bar, 0) ? 1u : 0u;
        out[1] = rz::PackBf16x2::execute(1.0f, 2.0f);
        out[2] = rz::PackE4m3x4::execute(1.0f, 2.0f, 500.0f, -500.0f);
        out[3] = rz::causal_tile_skip(0, 128, 128) ? 1u : 0u;
        float acc[2] = {1.0f, 2.0f};
        const uint32_t partial[2] = {0x3f800000u, 0x40000000u};
        iro::util::front_t<PromoteBound::realization::leaves>::execute(acc, partial, 0.5f);      // acc = {1.5, 3}
        out[4] = __float_as_uint(acc[0] + acc[1]);
    }
}
