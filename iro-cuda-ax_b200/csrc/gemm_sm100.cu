// sm_100a GEMM kernels behind axp_sm100_gemm_fp8_blockscaled / axp_sm100_gemm_bf16.
//
// Recipe realised (reference include/axp/level3/gemm.hpp:1075-2027, dataflow
// :1316-1585): per output tile, a K loop of  stage-issue -> wait -> MMA -> commit
// with fp32 accumulation of one partial per K tile, then cast to Recipe::out and
// store.  The reference leaves tile scheduling, the runtime K loop and the global
// store to the user's kernel; this file is that kernel.
//
// Structure (persistent, one CTA per SM):
//   warp 0      TMA producer: per stage a [128 rows x 128 B] A box and a
//               [256/G rows x 128 B] B box (G = CTAs per MMA), 128-byte swizzle,
//               ring of full/empty mbarriers
//   warp 1      tcgen05.mma issuer (one elected lane of the leader CTA); owns the
//               TMEM allocation (512 columns = two 128x256 fp32 accumulator stages)
//   warps 4..   epilogue warpgroups: each owns a slice of the 256 tile columns,
//               thread = one accumulator row (TMEM lane)
// G = 1: the CTA computes a 128 x 256 tile.  G = 2 (cta_group::2): a cluster of
// two CTAs computes a 256 x 256 tile; each CTA loads its own 128 rows of A and
// its own 128 rows of B (every TMA load has one destination CTA), the leader's
// full barrier collects both CTAs' transaction bytes, the leader issues one
// M = 256 MMA that reads both CTAs' shared memory, and each CTA keeps the
// accumulator rows of its own A half in its own tensor memory.
// BF16: the accumulator of a tile stays in TMEM for the whole K loop; the
//       epilogue of tile i overlaps the mainloop of tile i+1 (two TMEM stages).
// FP8 block-scaled: each 128-wide K block is accumulated into a fresh TMEM stage;
//       the epilogue warps promote it into fp32 registers with
//       acc += (sA[m,kb]*sB[n/128,kb]) * partial  while the tensor core works on
//       the next K block in the other TMEM stage.
#include <cuda_bf16.h>

#include "axp/realize/sm100.hpp"
#include "host_common.hpp"
#include "kernel_config.hpp"

namespace rz = axp::realize::sm100;

namespace {

constexpr int kBM = 128;                       // accumulator rows per CTA
constexpr int kBN = 256;
constexpr int kRowBytes = 128;                 // bytes of K per stage row (one swizzle span)
constexpr int kABytes = kBM * kRowBytes;       // 16 KiB
constexpr int kTmemCols = 512;
constexpr int kAccCols = kBN;                  // columns per accumulator stage
constexpr int kMaxStages = 6;
constexpr int kDefaultFp8TileN = 256;

template <int kCtaGroup>
struct StageCfg {
    static constexpr int kBRows = kBN / kCtaGroup;
    static constexpr int kBBytes = kBRows * kRowBytes;           // 32 or 16 KiB
    static constexpr int kStageBytes = kABytes + kBBytes;        // 48 or 32 KiB
    static constexpr int kStages = kCtaGroup == 1 ? 4 : 6;
    static constexpr int kDynSmem = kStages * kStageBytes + 1024;
};

// the default dispatch (launch_gemm) and the configuration header agree
namespace cfg = axp_shim::cfg;
static_assert(cfg::kGemmFp8.tile_m == kBM && cfg::kGemmFp8.tile_n == kBN && cfg::kGemmFp8.tile_k == kRowBytes);
static_assert(cfg::kGemmBf16.tile_m == kBM && cfg::kGemmBf16.tile_n == kBN && cfg::kGemmBf16.tile_k * 2 == kRowBytes);
static_assert(cfg::kGemmFp8.stages == StageCfg<cfg::kGemmFp8.cta_group>::kStages && cfg::kGemmFp8.stage_bytes == StageCfg<cfg::kGemmFp8.cta_group>::kStageBytes &&
              cfg::kGemmFp8.dyn_smem == StageCfg<cfg::kGemmFp8.cta_group>::kDynSmem && cfg::kGemmFp8.tmem_cols == kTmemCols);
static_assert(cfg::kGemmBf16.stages == StageCfg<cfg::kGemmBf16.cta_group>::kStages && cfg::kGemmBf16.stage_bytes == StageCfg<cfg::kGemmBf16.cta_group>::kStageBytes &&
              cfg::kGemmBf16.dyn_smem == StageCfg<cfg::kGemmBf16.cta_group>::kDynSmem && cfg::kGemmBf16.tmem_cols == kTmemCols);

struct GemmParams {
    const float* sA;      // [M, KB]
    const float* sB;      // [*, KB], row (sb_row0 + n/128)
    const float* sB2;     // gated FP8: block scales of the "up" weight, same layout as sB
    __nv_bfloat16* C;     // already offset to column n_begin
    int M;
    int N;                // local column count (n_end - n_begin)
    int k_blocks;         // ceil(K / elements per stage row)
    int scale_ld;         // K/128 (fp8 only)
    int sb_row0;          // n_begin / 128
    const float* bias;    // fused epilogue: per output column, already offset to column n_begin; null = none
    int act;              // fused epilogue activation after the bias add: 0 = identity, 1 = SiLU
    const __nv_bfloat16* c_in;   // linear-combination epilogue: out = alpha * acc + beta * c_in (offset to column n_begin); null = none
    long long ldcin;
    float alpha;
    float beta;
    long long ldc;
    uint32_t* status;
    // gated FP8 with a quantising epilogue: H leaves as E4M3 bytes plus one fp32 scale per row and 128 output columns
    // (the A operand and 1x128 scales of the next block-scaled GEMM) instead of bf16; null = bf16 output
    uint8_t* q_out;       // already offset to column n_begin
    float* q_scales;      // already offset to scale block n_begin / 128
    long long ldq;
    int q_scale_ld;       // scale blocks per row of the full output (N / 128)
#if defined(AXP_SM100_LATENCY_PROBES)
    unsigned long long* debug;   // timestamp buffer of the latency experiments
    int experiment;       // bit 0: skip the promotion arithmetic, bit 1: skip the tensor-memory reads (results invalid; times only)
#endif
};

// Parts of the epilogue can be switched off in builds with -DAXP_SM100_LATENCY_PROBES only; the production kernels and
// their parameter block carry none of it.
#if defined(AXP_SM100_LATENCY_PROBES)
#define AXP_GEMM_EXPERIMENT(p, mask) (((p).experiment & (mask)) != 0)
#else
#define AXP_GEMM_EXPERIMENT(p, mask) false
#endif

struct Pipe {
    uint64_t full[kMaxStages];
    uint64_t empty[kMaxStages];
    uint64_t tmem_full[2];
    uint64_t tmem_empty[2];
    uint64_t amax_ready;          // quantising epilogue: both warpgroups have published their half-block maxima
    float amax_half[2][2][kBM];   // [tile parity][warpgroup][row]
    uint32_t tmem_base;
    uint32_t abort_flag;
};

// Smallest block scale of the quantising epilogue, as in the stand-alone quantiser: the smallest normal float.
constexpr float kMinBlockScale = 1.17549435e-38f;

__device__ __forceinline__ void report(const GemmParams& p, Pipe* pipe, uint32_t code) {
    *reinterpret_cast<volatile uint32_t*>(&pipe->abort_flag) = 1u;
    if (p.status) atomicOr(p.status, rz::kStatusError | code);
}

__device__ __forceinline__ unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Latency probes exist only in builds with -DAXP_SM100_LATENCY_PROBES: CTA 0 stamps event `what`
// (0..3) of its first 64 K blocks; the production kernels carry none of it.
__device__ __forceinline__ void stamp(const GemmParams& p, int what, int n) {
#if defined(AXP_SM100_LATENCY_PROBES)
    if (p.debug && blockIdx.x == 0 && n < 64) atomicMax(&p.debug[what * 64 + n], global_timer_ns());
#else
    (void)p; (void)what; (void)n;
#endif
}

// The fused epilogues (bias + activation, linear combination, gated) are the kit's BiasActFma leaf, the promotion of a
// K-block partial its ScalePromoteFma leaf, the 16-byte row stores its RowStoreVec16 leaf (include/axp/realize/sm100.hpp).
// Tile order: groups of kGroup row tiles sweep all column tiles, so that the CTAs
// running at one time share a few A row panels and B column panels in L2.
// Row tiles (of 128 rows) that share one sweep over the column tiles: the tiles the 148 CTAs work on at a time then touch
// kTileGroup A row blocks and ~148 / kTileGroup B column blocks, which L2 holds.  Measured on 8192^3 FP8 / the bf16 MLP
// gate/up shape: 8: 2016 / 1492, 16: 2005 / 1519, 32: 2078 / 1599, 64: 1874 / 1395, 128: 1877 / 1221 TFLOP/s.
constexpr int kTileGroup = 32;

template <int kGroup>
__device__ __forceinline__ void tile_coords(int t, int num_m, int num_n, int& tm, int& tn) {
    const int per_group = kGroup * num_n;
    const int g = t / per_group;
    const int r = t - g * per_group;
    const int rows = min(kGroup, num_m - g * kGroup);
    tm = g * kGroup + r % rows;
    tn = r / rows;
}

// kEpiWG epilogue warpgroups split the 256 tile columns between them; kCtaGroup
// CTAs cooperate on one MMA.
// kGated (bf16, four epilogue warpgroups): the B tile of a stage is 128 rows of a "gate" weight followed by
// the same 128 rows of an "up" weight (second tensor map), so that accumulator columns [0,128) hold X.Wg^T and
// [128,256) hold X.Wu^T of the same 128 output columns, and the epilogue writes SiLU(gate) * up: the gate / up
// projection of a gated MLP in one pass, without the two intermediate matrices ever reaching HBM.
template <bool kFp8, int kEpiWG, int kCtaGroup, bool kGated = false>
__global__ void __launch_bounds__(128 * (1 + kEpiWG), 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
            const __grid_constant__ CUtensorMap tmB2, const GemmParams p) {
    static_assert(!kGated || (!kFp8 && kEpiWG == 4) || (kFp8 && kEpiWG == 2),
                  "the gated epilogue exists for bf16 with four epilogue warpgroups and for FP8 with two");
    constexpr int kOutN = kGated ? kBN / 2 : kBN;     // output columns per tile
    using SC = StageCfg<kCtaGroup>;
    constexpr int kStages = SC::kStages;
    constexpr int kStageBytes = SC::kStageBytes;
    constexpr int kCols = kBN / kEpiWG;               // accumulator columns per epilogue thread
    constexpr int kChunks = kCols / 32;
    constexpr int kEpilogueWarps = 4 * kEpiWG;
    // setmaxnreg only moves registers inside the CTA's launch allocation (threads x launch
    // registers): an increase that the decreases do not cover would block forever.
    constexpr int kThreads = 128 * (1 + kEpiWG);
    constexpr int kLaunchRegs = (65536 / kThreads) / 8 * 8;          // 168 or 96
    constexpr int kProducerRegs = kEpiWG == 2 ? 40 : 32;
    constexpr int kEpilogueRegs = kEpiWG == 2 ? 232 : 112;
    static_assert(128 * kProducerRegs + 128 * kEpiWG * kEpilogueRegs <= kThreads * kLaunchRegs,
                  "register budgets exceed the CTA's launch allocation");
    static_assert(kEpiWG != 2 || (kProducerRegs == cfg::kGemmFp8.producer_regs && kEpilogueRegs == cfg::kGemmFp8.epilogue_regs && kThreads == cfg::kGemmFp8.threads));
    static_assert(kEpiWG != 4 || (kProducerRegs == cfg::kGemmBf16.producer_regs && kEpilogueRegs == cfg::kGemmBf16.epilogue_regs && kThreads == cfg::kGemmBf16.threads));
    constexpr int kElemsPerRow = kFp8 ? 128 : 64;     // K elements per stage
    constexpr int kMmaPerStage = kRowBytes / 32;      // one MMA consumes 32 bytes of K
    constexpr int kTileM = kBM * kCtaGroup;           // rows of the (pair) tile
    constexpr uint32_t kFmt = kFp8 ? 0u : 1u;         // e4m3 / bf16
    // One N = 256 MMA per 32 bytes of K.  (Issuing each K block as two N = 128 halves with four
    // half-stages in flight was measured slower: the A tile is then fetched from shared memory twice.)
    constexpr uint32_t kIdesc = rz::make_instr_desc(kFmt, kFmt, false, false, kTileM, kBN);

    extern __shared__ uint8_t dyn_smem_raw[];
    __shared__ Pipe pipe;

    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(dyn_smem_raw) + 1023) & ~uintptr_t(1023));
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    volatile uint32_t* abort_flag = &pipe.abort_flag;
    const uint32_t cta_rank = (kCtaGroup == 2) ? rz::cluster_cta_rank() : 0u;
    const bool leader = cta_rank == 0;

    const int num_m = (p.M + kTileM - 1) / kTileM;
    const int num_n = (p.N + kOutN - 1) / kOutN;
    const int num_tiles = num_m * num_n;
    const int first_tile = int(blockIdx.x) / kCtaGroup;
    const int tile_step = int(gridDim.x) / kCtaGroup;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            rz::BarrierInit::execute(&pipe.full[s], 1);
            rz::BarrierInit::execute(&pipe.empty[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            rz::BarrierInit::execute(&pipe.tmem_full[a], 1);
            rz::BarrierInit::execute(&pipe.tmem_empty[a], kEpilogueWarps * kCtaGroup);
        }
        rz::BarrierInit::execute(&pipe.amax_ready, kEpilogueWarps);
        pipe.abort_flag = 0;
        rz::BarrierInitFence::execute();
    }
    if constexpr (kCtaGroup == 2) rz::ClusterSync::execute();   // the peer's barriers exist before anything signals them
    if (warp == 1) rz::TmemAlloc<kCtaGroup>::execute(&pipe.tmem_base, kTmemCols);
    rz::Tcgen05FenceBefore::execute();
    __syncthreads();
    rz::Tcgen05FenceAfter::execute();
    const uint32_t tmem_base = pipe.tmem_base;

    if (warp < 4) {
        rz::RegDealloc<kProducerRegs>::execute();
        if (warp == 0) {
            // ------------------------------------------------ TMA producer ----
            // the whole warp runs the loop (waits are votes of all lanes), one elected lane issues the copies
            {
                const bool elected = rz::elect_one();
                if (elected) {
                    rz::PrefetchTensorMap::execute(&tmA);
                    rz::PrefetchTensorMap::execute(&tmB);
                    if constexpr (kGated) rz::PrefetchTensorMap::execute(&tmB2);
                }
                int stage = 0;
                uint32_t phase = 0;
                bool ok = true;
                for (int t = first_tile; t < num_tiles && ok; t += tile_step) {
                    int tm, tn;
                    tile_coords<kTileGroup / kCtaGroup>(t, num_m, num_n, tm, tn);
                    const int a_row = tm * kTileM + int(cta_rank) * kBM;
                    const int b_row = kGated ? tn * kOutN : tn * kBN + int(cta_rank) * SC::kBRows;
                    for (int kb = 0; kb < p.k_blocks; ++kb) {
                        if (!__all_sync(0xffffffffu, rz::BarrierWait::execute(&pipe.empty[stage], phase ^ 1u, abort_flag))) {
                            if (elected) report(p, &pipe, rz::kRoleProducer | rz::kBarEmpty);
                            ok = false;
                            break;
                        }
                        uint8_t* sa = smem + stage * kStageBytes;
                        uint8_t* sb = sa + kABytes;
                        if (!elected) {
                        } else if constexpr (kCtaGroup == 1) {
                            rz::BarrierExpectTx::execute(&pipe.full[stage], kStageBytes);
                            rz::BulkTmaCopy2D::execute(&tmA, sa, kb * kElemsPerRow, a_row, &pipe.full[stage]);
                            if constexpr (kGated) {
                                rz::BulkTmaCopy2D::execute(&tmB, sb, kb * kElemsPerRow, b_row, &pipe.full[stage]);
                                rz::BulkTmaCopy2D::execute(&tmB2, sb + (kBN / 2) * kRowBytes, kb * kElemsPerRow, b_row, &pipe.full[stage]);
                            } else {
                                rz::BulkTmaCopy2D::execute(&tmB, sb, kb * kElemsPerRow, b_row, &pipe.full[stage]);
                            }
                        } else {
                            // both CTAs' bytes are counted on the leader's barrier
                            if (leader) rz::BarrierExpectTx::execute(&pipe.full[stage], 2 * kStageBytes);
                            rz::BulkTmaCopy2DPeerBarrier::execute(&tmA, sa, kb * kElemsPerRow, a_row, &pipe.full[stage], 0);
                            // gated: the leader holds the gate rows, its peer the up rows of the same output columns
                            rz::BulkTmaCopy2DPeerBarrier::execute((kGated && !leader) ? &tmB2 : &tmB, sb, kb * kElemsPerRow, b_row,
                                                                  &pipe.full[stage], 0);
                        }
                        if (++stage == kStages) { stage = 0; phase ^= 1u; }
                    }
                }
                // tail: every slot must have been released before shared memory goes away
                for (int s = 0; s < kStages && ok; ++s) {
                    if (!__all_sync(0xffffffffu, rz::BarrierWait::execute(&pipe.empty[stage], phase ^ 1u, abort_flag))) {
                        if (elected) report(p, &pipe, rz::kRoleProducer | rz::kBarEmpty);
                        ok = false;
                    }
                    if (++stage == kStages) { stage = 0; phase ^= 1u; }
                }
            }
        } else if (warp == 1) {
            // -------------------------------------------------- MMA issuer ----
            // The whole warp runs the loop (every wait is a vote of all lanes) and one elected lane issues: loop control
            // and descriptor arithmetic stay warp-uniform, which makes the issue cheaper beside the busy epilogue warps.
            if (leader) {
                const bool elected = rz::elect_one();
                int stage = 0;
                uint32_t phase = 0;
                int acc = 0;
                uint32_t acc_phase = 0;
                bool ok = true;
                int n_dbg = 0;
                auto commit = [&](uint64_t* bar) {
                    if constexpr (kCtaGroup == 1) rz::Tcgen05Commit<1>::execute(bar);
                    else rz::Tcgen05CommitPair::execute(bar, uint16_t(3));    // same barrier in both CTAs
                };
                for (int t = first_tile; t < num_tiles && ok; t += tile_step) {
                    if constexpr (!kFp8) {
                        if (!__all_sync(0xffffffffu, rz::BarrierWait::execute(&pipe.tmem_empty[acc], acc_phase ^ 1u, abort_flag))) {
                            if (elected) report(p, &pipe, rz::kRoleMma | rz::kBarTmemEmpty);
                            ok = false;
                            break;
                        }
                    }
                    for (int kb = 0; kb < p.k_blocks; ++kb) {
                        if constexpr (kFp8) {
                            if (!__all_sync(0xffffffffu, rz::BarrierSpinWait::execute(&pipe.tmem_empty[acc], acc_phase ^ 1u, abort_flag))) {
                                if (elected) report(p, &pipe, rz::kRoleMma | rz::kBarTmemEmpty);
                                ok = false;
                                break;
                            }
                        }
                        if (elected) stamp(p, 0, n_dbg);      // accumulator stage released to the issuer
                        if (!__all_sync(0xffffffffu, rz::BarrierWait::execute(&pipe.full[stage], phase, abort_flag))) {
                            if (elected) report(p, &pipe, rz::kRoleMma | rz::kBarFull);
                            ok = false;
                            break;
                        }
                        if (elected) stamp(p, 1, n_dbg);      // operands present
                        rz::Tcgen05FenceAfter::execute();
                        const uint32_t sa = rz::smem_u32(smem + stage * kStageBytes);
                        const uint64_t da = rz::MakeSmemDescKMajorSw128::execute(sa);
                        const uint64_t db = rz::MakeSmemDescKMajorSw128::execute(sa + kABytes);
                        const uint32_t d_tmem = tmem_base + uint32_t(acc * kAccCols);
                        if (elected) {
#pragma unroll
                            for (int k = 0; k < kMmaPerStage; ++k) {
                                const uint32_t accumulate = kFp8 ? uint32_t(k > 0) : uint32_t((kb | k) != 0);
                                // +32 bytes of K per step = +2 in the descriptor's 16-byte units
                                rz::Tcgen05Mma<kCtaGroup, !kFp8>::execute(d_tmem, da + uint64_t(2 * k), db + uint64_t(2 * k),
                                                                          kIdesc, accumulate);
                            }
                        }
                        if constexpr (kFp8) {
                            if (elected) commit(&pipe.tmem_full[acc]);       // the epilogue is on the critical path: tell it first
                            if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
                        }
                        if (elected) commit(&pipe.empty[stage]);
                        if (++stage == kStages) { stage = 0; phase ^= 1u; }
                        ++n_dbg;
                    }
                    if constexpr (!kFp8) {
                        if (ok) {
                            if (elected) commit(&pipe.tmem_full[acc]);
                            if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
                        }
                    }
                }
            }
        }
    } else {
        // ---------------------------------------------------- epilogue ----
        rz::RegAlloc<kEpilogueRegs>::execute();
        const int ewarp = warp - 4;
        const int g = ewarp >> 2;              // which column slice of the tile
        const int quarter = warp & 3;          // TMEM lane quarter this warp may touch
        const int row_in_tile = quarter * 32 + lane;
        const uint32_t lane_addr = uint32_t(quarter * 32) << 16;
        int acc = 0;
        uint32_t acc_phase = 0;
        bool ok = true;
        int n_dbg = 0;
        int tile_count = 0;      // tiles this CTA has finished (quantising epilogue: parity of the exchange)
        // the accumulator stage goes back to the leader's MMA issuer
        auto release_acc = [&](uint64_t* bar) {
            // the hand-over publishes no generic-proxy memory (the tensor-memory reads have completed), so the remote
            // arrive needs no release ordering, which would cost several hundred cycles per arrive
            if constexpr (kCtaGroup == 1) rz::BarrierArrive::execute(bar);
            else rz::ClusterBarrierArriveRelaxed::execute(bar, 0);
        };
        for (int t = first_tile; t < num_tiles && ok; t += tile_step) {
            int tm, tn;
            tile_coords<kTileGroup / kCtaGroup>(t, num_m, num_n, tm, tn);
            const int row = tm * kTileM + int(cta_rank) * kBM + row_in_tile;
            const int col0 = tn * kBN + g * kCols;
            const bool row_ok = row < p.M;
            __nv_bfloat16* crow = p.C + (long long)row * p.ldc + col0;
            if constexpr (kFp8) {
                // Gated: the accumulator holds gate columns [0,128) and up columns [128,256) of the same 128 outputs; this
                // thread promotes gate columns [64 g, +64) into accum[0..63] and the matching up columns into accum[64..127].
                const int ocol0 = kGated ? tn * kOutN + g * (kCols / 2) : col0;         // first output column of this thread
                float accum[kCols];
#pragma unroll
                for (int j = 0; j < kCols; ++j) accum[j] = 0.0f;
                const float* sa_row = p.sA + (long long)(row_ok ? row : 0) * p.scale_ld;
                const bool col_ok = ocol0 < p.N;
                const long long sb_off = (long long)(p.sb_row0 + (col_ok ? ocol0 : 0) / 128) * p.scale_ld;
                const float* sb_row = p.sB + sb_off;
                const float* sb2_row = kGated ? p.sB2 + sb_off : sb_row;
                float s_next = __ldg(sa_row) * __ldg(sb_row);
                float s2_next = kGated ? __ldg(sa_row) * __ldg(sb2_row) : 0.0f;
                for (int kb = 0; kb < p.k_blocks; ++kb) {
                    const float s = s_next;
                    const float s2 = s2_next;
                    if (kb + 1 < p.k_blocks) {      // hidden behind this block
                        s_next = __ldg(sa_row + kb + 1) * __ldg(sb_row + kb + 1);
                        if constexpr (kGated) s2_next = __ldg(sa_row + kb + 1) * __ldg(sb2_row + kb + 1);
                    }
                    if (!rz::BarrierWait::execute(&pipe.tmem_full[acc], acc_phase, abort_flag)) {
                        if (lane == 0) report(p, &pipe, rz::kRoleEpilogue | rz::kBarTmemFull);
                        ok = false;
                        break;
                    }
                    if (lane == 0) stamp(p, 2, n_dbg);      // partial accumulator seen by the epilogue
                    rz::Tcgen05FenceAfter::execute();
                    const uint32_t tstage = tmem_base + lane_addr + uint32_t(acc * kAccCols);
                    // chunk c (32 columns) of this thread: plain = consecutive columns of its slice; gated = two gate chunks,
                    // then the two up chunks 128 columns further
                    auto chunk_addr = [&](int c) {
                        if constexpr (kGated) return tstage + uint32_t((c / 2) * (kBN / 2) + g * (kCols / 2) + (c % 2) * 32);
                        else return tstage + uint32_t(g * kCols + c * 32);
                    };
                    // TMEM reads run one chunk ahead of the arithmetic; the stage goes back to the
                    // issuer as soon as the last read has landed, before the last chunk's FMAs
                    uint32_t va[32], vb[32];
                    auto promote = [&](const uint32_t (&v)[32], int c) {
                        if (!AXP_GEMM_EXPERIMENT(p, 1)) {
                            const float sc = (kGated && c >= kChunks / 2) ? s2 : s;
                            rz::ScalePromoteFma::execute(&accum[c * 32], v, sc);
                        }
                    };
                    if (!AXP_GEMM_EXPERIMENT(p, 2)) {
                        rz::TmemLoad32x32::execute(chunk_addr(0), va);
                        rz::TmemLoadWait::execute(va);
#pragma unroll
                        for (int c = 0; c < kChunks; c += 2) {
                            rz::TmemLoad32x32::execute(chunk_addr(c + 1), vb);
                            promote(va, c);
                            rz::TmemLoadWait::execute(vb);
                            if (c + 2 < kChunks) {
                                rz::TmemLoad32x32::execute(chunk_addr(c + 2), va);
                                promote(vb, c + 1);
                                rz::TmemLoadWait::execute(va);
                            }
                        }
                    }
                    rz::Tcgen05FenceBefore::execute();
                    __syncwarp();
                    if (lane == 0) release_acc(&pipe.tmem_empty[acc]);
                    if (!AXP_GEMM_EXPERIMENT(p, 2)) promote(vb, kChunks - 1);
                    if (lane == 0) stamp(p, 3, n_dbg);   // this warp's release issued
                    ++n_dbg;
                    if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
                }
                if constexpr (kGated) {
                    if (p.q_out != nullptr) {
                        // Quantising epilogue: the bf16 values this kernel would have stored are quantised in registers exactly
                        // as the stand-alone quantiser would quantise them (block maximum / 448, IEEE divisions, saturating
                        // E4M3 conversion).  The 128-column scale block of a row is this tile's whole output row: its two
                        // halves belong to the row's threads in the two warpgroups, which exchange their maxima through
                        // shared memory behind an mbarrier (bounded wait, like every other wait of the kernel).
                        if (!ok) break;
                        uint32_t hw[kCols / 4];
                        float amax = 0.0f;
#pragma unroll
                        for (int i = 0; i < kCols / 4; ++i) {
                            hw[i] = rz::BiasActFma::gated(accum[2 * i], accum[2 * i + 1], accum[kCols / 2 + 2 * i], accum[kCols / 2 + 2 * i + 1]);
                            if (ocol0 + 2 * i < p.N)
                                amax = fmaxf(amax, fmaxf(fabsf(__uint_as_float(hw[i] << 16)), fabsf(__uint_as_float(hw[i] & 0xffff0000u))));
                        }
                        const int par = tile_count & 1;
                        pipe.amax_half[par][g][row_in_tile] = amax;
                        __syncwarp();
                        if (lane == 0) rz::BarrierArrive::execute(&pipe.amax_ready);
                        if (!rz::BarrierWait::execute(&pipe.amax_ready, uint32_t(tile_count & 1), abort_flag)) {
                            if (lane == 0) report(p, &pipe, rz::kRoleEpilogue | rz::kBarOther);
                            ok = false;
                            break;
                        }
                        amax = fmaxf(amax, pipe.amax_half[par][g ^ 1][row_in_tile]);
                        const float scale = amax > 0.0f ? fmaxf(__fdiv_rn(amax, 448.0f), kMinBlockScale) : 1.0f;
                        const float inv = __fdiv_rn(1.0f, scale);
                        if (row_ok && ocol0 < p.N) {
                            uint8_t* qrow = p.q_out + (long long)row * p.ldq + ocol0;
#pragma unroll
                            for (int c = 0; c < kCols / 32; ++c) {      // 16 outputs = 16 bytes per store
                                uint32_t q[4];
#pragma unroll
                                for (int i = 0; i < 4; ++i) {
                                    const uint32_t w0 = hw[c * 8 + 2 * i], w1 = hw[c * 8 + 2 * i + 1];
                                    q[i] = rz::PackE4m3x4::execute(__uint_as_float(w0 << 16) * inv, __uint_as_float(w0 & 0xffff0000u) * inv,
                                                                   __uint_as_float(w1 << 16) * inv, __uint_as_float(w1 & 0xffff0000u) * inv);
                                }
                                *reinterpret_cast<uint4*>(qrow + c * 16) = make_uint4(q[0], q[1], q[2], q[3]);
                            }
                            if (g == 0) p.q_scales[(long long)row * p.q_scale_ld + tn] = scale;
                        }
                        ++tile_count;
                    } else if (ok && row_ok) {
                        __nv_bfloat16* orow = p.C + (long long)row * p.ldc + ocol0;
#pragma unroll
                        for (int c = 0; c < kCols / 16; ++c) {
                            if (ocol0 + c * 8 < p.N) {
                                uint32_t o[4];
#pragma unroll
                                for (int i = 0; i < 4; ++i) {
                                    const float g0 = accum[c * 8 + 2 * i], g1 = accum[c * 8 + 2 * i + 1];
                                    const float u0 = accum[kCols / 2 + c * 8 + 2 * i], u1 = accum[kCols / 2 + c * 8 + 2 * i + 1];
                                    o[i] = rz::BiasActFma::gated(g0, g1, u0, u1);
                                }
                                rz::RowStoreVec16::execute(orow + c * 8, make_uint4(o[0], o[1], o[2], o[3]));
                            }
                        }
                    }
                } else if (ok && row_ok) {
                    bool stored = false;
                    if constexpr (kCols == 128) {
                        if (p.q_out != nullptr) {
                            // Quantising epilogue: a thread's 128 columns are one scale block of its row.  The bf16 values the
                            // plain epilogue would store (bias, activation, linear combination included) are quantised in
                            // registers exactly as the stand-alone quantiser would quantise them.
                            stored = true;
                            uint4 w[kCols / 8];
                            float amax = 0.0f;
#pragma unroll
                            for (int c = 0; c < kCols / 8; ++c) {
                                float f[8];
#pragma unroll
                                for (int i = 0; i < 8; ++i) f[i] = accum[c * 8 + i];
                                w[c] = rz::BiasActFma::execute(f, p.bias ? p.bias + col0 + c * 8 : nullptr, p.act,
                                        p.c_in ? p.c_in + (long long)row * p.ldcin + col0 + c * 8 : nullptr, p.alpha, p.beta);
                                const uint32_t ww[4] = {w[c].x, w[c].y, w[c].z, w[c].w};
#pragma unroll
                                for (int i = 0; i < 4; ++i)
                                    amax = fmaxf(amax, fmaxf(fabsf(__uint_as_float(ww[i] << 16)), fabsf(__uint_as_float(ww[i] & 0xffff0000u))));
                            }
                            const float scale = amax > 0.0f ? fmaxf(__fdiv_rn(amax, 448.0f), kMinBlockScale) : 1.0f;
                            const float inv = __fdiv_rn(1.0f, scale);
                            if (col0 < p.N) {
                                uint8_t* qrow = p.q_out + (long long)row * p.ldq + col0;
#pragma unroll
                                for (int c = 0; c < kCols / 16; ++c) {      // 16 outputs = 16 bytes per store
                                    const uint32_t ww[8] = {w[2 * c].x, w[2 * c].y, w[2 * c].z, w[2 * c].w, w[2 * c + 1].x, w[2 * c + 1].y, w[2 * c + 1].z, w[2 * c + 1].w};
                                    uint32_t q[4];
#pragma unroll
                                    for (int i = 0; i < 4; ++i)
                                        q[i] = rz::PackE4m3x4::execute(__uint_as_float(ww[2 * i] << 16) * inv, __uint_as_float(ww[2 * i] & 0xffff0000u) * inv,
                                                                       __uint_as_float(ww[2 * i + 1] << 16) * inv, __uint_as_float(ww[2 * i + 1] & 0xffff0000u) * inv);
                                    *reinterpret_cast<uint4*>(qrow + c * 16) = make_uint4(q[0], q[1], q[2], q[3]);
                                }
                                p.q_scales[(long long)row * p.q_scale_ld + tn * (kBN / 128) + g] = scale;
                            }
                        }
                    }
                    if (!stored) {
#pragma unroll
                        for (int c = 0; c < kCols / 8; ++c) {
                            if (col0 + c * 8 < p.N) {
                                float f[8];
#pragma unroll
                                for (int i = 0; i < 8; ++i) f[i] = accum[c * 8 + i];
                                rz::RowStoreVec16::execute(crow + c * 8,
                                    rz::BiasActFma::execute(f, p.bias ? p.bias + col0 + c * 8 : nullptr, p.act,
                                            p.c_in ? p.c_in + (long long)row * p.ldcin + col0 + c * 8 : nullptr, p.alpha, p.beta));
                            }
                        }
                    }
                }
            } else if constexpr (kGated) {
                if (!rz::BarrierWait::execute(&pipe.tmem_full[acc], acc_phase, abort_flag)) {
                    if (lane == 0) report(p, &pipe, rz::kRoleEpilogue | rz::kBarTmemFull);
                    ok = false;
                    break;
                }
                rz::Tcgen05FenceAfter::execute();
                // this warpgroup's 32 output columns: gate at accumulator columns [32g, 32g+32), up 128 columns further
                const uint32_t taddr = tmem_base + lane_addr + uint32_t(acc * kAccCols + g * 32);
                const int ocol = tn * kOutN + g * 32;
                uint32_t vg[32], vu[32];
                rz::TmemLoad32x32::execute(taddr, vg);
                rz::TmemLoad32x32::execute(taddr + uint32_t(kBN / 2), vu);
                rz::TmemLoadWait::execute(vg);
                rz::TmemLoadWait::execute(vu);
                rz::Tcgen05FenceBefore::execute();
                __syncwarp();
                if (lane == 0) release_acc(&pipe.tmem_empty[acc]);      // both chunks are in registers: free the stage early
                if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
                if (row_ok) {
                    __nv_bfloat16* orow = p.C + (long long)row * p.ldc + ocol;
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        if (ocol + q * 8 < p.N) {
                            uint32_t o[4];
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                const float g0 = __uint_as_float(vg[q * 8 + 2 * i]), g1 = __uint_as_float(vg[q * 8 + 2 * i + 1]);
                                const float u0 = __uint_as_float(vu[q * 8 + 2 * i]), u1 = __uint_as_float(vu[q * 8 + 2 * i + 1]);
                                o[i] = rz::BiasActFma::gated(g0, g1, u0, u1);
                            }
                            rz::RowStoreVec16::execute(orow + q * 8, make_uint4(o[0], o[1], o[2], o[3]));
                        }
                    }
                }
            } else {
                if (!rz::BarrierWait::execute(&pipe.tmem_full[acc], acc_phase, abort_flag)) {
                    if (lane == 0) report(p, &pipe, rz::kRoleEpilogue | rz::kBarTmemFull);
                    ok = false;
                    break;
                }
                rz::Tcgen05FenceAfter::execute();
                const uint32_t taddr = tmem_base + lane_addr + uint32_t(acc * kAccCols + g * kCols);
#pragma unroll
                for (int c = 0; c < kChunks; ++c) {
                    uint32_t v[32];
                    rz::TmemLoad32x32::execute(taddr + uint32_t(c * 32), v);
                    rz::TmemLoadWait::execute();
                    if (row_ok) {
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            if (col0 + c * 32 + q * 8 < p.N) {
                                float f[8];
#pragma unroll
                                for (int i = 0; i < 8; ++i) f[i] = __uint_as_float(v[q * 8 + i]);
                                rz::RowStoreVec16::execute(crow + c * 32 + q * 8,
                                    rz::BiasActFma::execute(f, p.bias ? p.bias + col0 + c * 32 + q * 8 : nullptr, p.act,
                                            p.c_in ? p.c_in + (long long)row * p.ldcin + col0 + c * 32 + q * 8 : nullptr, p.alpha, p.beta));
                            }
                        }
                    }
                }
                rz::Tcgen05FenceBefore::execute();
                __syncwarp();
                if (lane == 0) release_acc(&pipe.tmem_empty[acc]);
                if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
            }
        }
    }

    rz::Tcgen05FenceBefore::execute();
    __syncthreads();
    if constexpr (kCtaGroup == 2) rz::ClusterSync::execute();   // the peer no longer touches this CTA's barriers or TMEM
    if (warp == 1) {
        rz::Tcgen05FenceAfter::execute();
        rz::TmemDealloc<kCtaGroup>::execute(tmem_base, kTmemCols);
    }
}

// ----------------------------------------------------------------------------
// FP8 block-scaled GEMM, 128 x 128 tiles, TWO CTAs per SM.
// The 128 x 256 kernel above is bound by the accumulator hand-over that every 128-deep K block needs
// (tensor core -> epilogue -> tensor core takes about three times as long as the MMAs of the block, with room
// for only two 128 x 256 accumulator stages in tensor memory).  Here a CTA owns 256 tensor-memory columns (two
// 128 x 128 stages) and 96 KiB of shared memory (three 32 KiB operand stages), so two CTAs share an SM: while
// one CTA's K block is handed over, the other CTA's MMAs run, and sixteen epilogue warps instead of eight hide the
// tensor-memory load latency.  384 threads: warp 0 producer, warp 1 issuer, warps 4-11 two epilogue warpgroups
// (thread = accumulator row, 64 columns each).
// ----------------------------------------------------------------------------
constexpr int kN128Stages = 3;
constexpr int kN128StageBytes = 2 * kABytes;                       // A 16 KiB + B 16 KiB
constexpr int kN128DynSmem = kN128Stages * kN128StageBytes + 1024;
constexpr int kN128TmemCols = 256;

__global__ void __launch_bounds__(384, 2)
gemm_fp8_n128_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const GemmParams p) {
    constexpr int kTileN = 128;
    constexpr int kCols = 64;                                    // accumulator columns per epilogue thread
    // two CTAs per SM: 65536 / 768 threads = 85 -> 80 registers at launch; setmaxnreg moves them inside the CTA
    constexpr int kLaunchRegs = 80, kProducerRegs = 32, kEpilogueRegs = 104;
    static_assert(128 * kProducerRegs + 256 * kEpilogueRegs <= 384 * kLaunchRegs, "register budgets exceed the CTA's launch allocation");
    constexpr uint32_t kIdesc = rz::make_instr_desc(0u, 0u, false, false, kBM, kTileN);

    extern __shared__ uint8_t dyn_smem_raw[];
    __shared__ Pipe pipe;
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(dyn_smem_raw) + 1023) & ~uintptr_t(1023));
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    volatile uint32_t* abort_flag = &pipe.abort_flag;
    const int num_m = (p.M + kBM - 1) / kBM;
    const int num_n = (p.N + kTileN - 1) / kTileN;
    const int num_tiles = num_m * num_n;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kN128Stages; ++s) {
            rz::BarrierInit::execute(&pipe.full[s], 1);
            rz::BarrierInit::execute(&pipe.empty[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            rz::BarrierInit::execute(&pipe.tmem_full[a], 1);
            rz::BarrierInit::execute(&pipe.tmem_empty[a], 8);     // one arrival per epilogue warp
        }
        pipe.abort_flag = 0;
        rz::BarrierInitFence::execute();
    }
    if (warp == 1) rz::TmemAlloc<1>::execute(&pipe.tmem_base, kN128TmemCols);
    rz::Tcgen05FenceBefore::execute();
    __syncthreads();
    rz::Tcgen05FenceAfter::execute();
    const uint32_t tmem_base = pipe.tmem_base;

    if (warp < 4) {
        rz::RegDealloc<kProducerRegs>::execute();
        if (warp == 0 && lane == 0) {
            // ------------------------------------------------ TMA producer ----
            rz::PrefetchTensorMap::execute(&tmA);
            rz::PrefetchTensorMap::execute(&tmB);
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
                int tm, tn;
                tile_coords<16>(t, num_m, num_n, tm, tn);
                for (int kb = 0; kb < p.k_blocks; ++kb) {
                    if (!rz::BarrierWait::execute(&pipe.empty[stage], phase ^ 1u, abort_flag)) {
                        report(p, &pipe, rz::kRoleProducer | rz::kBarEmpty);
                        ok = false;
                        break;
                    }
                    uint8_t* sa = smem + stage * kN128StageBytes;
                    rz::BarrierExpectTx::execute(&pipe.full[stage], kN128StageBytes);
                    rz::BulkTmaCopy2D::execute(&tmA, sa, kb * 128, tm * kBM, &pipe.full[stage]);
                    rz::BulkTmaCopy2D::execute(&tmB, sa + kABytes, kb * 128, tn * kTileN, &pipe.full[stage]);
                    if (++stage == kN128Stages) { stage = 0; phase ^= 1u; }
                }
            }
            // tail: every slot must have been released before shared memory goes away
            for (int s = 0; s < kN128Stages && ok; ++s) {
                if (!rz::BarrierWait::execute(&pipe.empty[stage], phase ^ 1u, abort_flag)) {
                    report(p, &pipe, rz::kRoleProducer | rz::kBarEmpty);
                    ok = false;
                }
                if (++stage == kN128Stages) { stage = 0; phase ^= 1u; }
            }
        } else if (warp == 1 && lane == 0) {
            // -------------------------------------------------- MMA issuer ----
            int stage = 0, acc = 0;
            uint32_t phase = 0, acc_phase = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
                for (int kb = 0; kb < p.k_blocks; ++kb) {
                    if (!rz::BarrierWait::execute(&pipe.tmem_empty[acc], acc_phase ^ 1u, abort_flag)) {
                        report(p, &pipe, rz::kRoleMma | rz::kBarTmemEmpty);
                        ok = false;
                        break;
                    }
                    if (!rz::BarrierWait::execute(&pipe.full[stage], phase, abort_flag)) {
                        report(p, &pipe, rz::kRoleMma | rz::kBarFull);
                        ok = false;
                        break;
                    }
                    rz::Tcgen05FenceAfter::execute();
                    const uint32_t sa = rz::smem_u32(smem + stage * kN128StageBytes);
                    const uint64_t da = rz::MakeSmemDescKMajorSw128::execute(sa);
                    const uint64_t db = rz::MakeSmemDescKMajorSw128::execute(sa + kABytes);
                    const uint32_t d_tmem = tmem_base + uint32_t(acc * kTileN);
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        rz::Tcgen05Mma<1, false>::execute(d_tmem, da + uint64_t(2 * k), db + uint64_t(2 * k), kIdesc, uint32_t(k > 0));
                    rz::Tcgen05Commit<1>::execute(&pipe.tmem_full[acc]);
                    if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
                    rz::Tcgen05Commit<1>::execute(&pipe.empty[stage]);
                    if (++stage == kN128Stages) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else {
        // ---------------------------------------------------- epilogue ----
        rz::RegAlloc<kEpilogueRegs>::execute();
        const int g = (warp - 4) >> 2;           // column half of the tile
        const int quarter = warp & 3;            // TMEM lane quarter this warp may touch
        const int row_in_tile = quarter * 32 + lane;
        const uint32_t lane_addr = uint32_t(quarter * 32) << 16;
        int acc = 0;
        uint32_t acc_phase = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
            int tm, tn;
            tile_coords<16>(t, num_m, num_n, tm, tn);
            const int row = tm * kBM + row_in_tile;
            const int col0 = tn * kTileN + g * kCols;
            const bool row_ok = row < p.M;
            float accum[kCols];
#pragma unroll
            for (int j = 0; j < kCols; ++j) accum[j] = 0.0f;
            const float* sa_row = p.sA + (long long)(row_ok ? row : 0) * p.scale_ld;
            const float* sb_row = p.sB + (long long)(p.sb_row0 + (col0 < p.N ? col0 : 0) / 128) * p.scale_ld;
            float s_next = __ldg(sa_row) * __ldg(sb_row);
            for (int kb = 0; kb < p.k_blocks; ++kb) {
                const float s = s_next;
                if (kb + 1 < p.k_blocks) s_next = __ldg(sa_row + kb + 1) * __ldg(sb_row + kb + 1);
                if (!rz::BarrierWait::execute(&pipe.tmem_full[acc], acc_phase, abort_flag)) {
                    if (lane == 0) report(p, &pipe, rz::kRoleEpilogue | rz::kBarTmemFull);
                    ok = false;
                    break;
                }
                rz::Tcgen05FenceAfter::execute();
                const uint32_t taddr = tmem_base + lane_addr + uint32_t(acc * kTileN + g * kCols);
                // four 16-column reads; the stage goes back to the issuer once the last one has landed
                uint32_t v[16];
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    rz::TmemLoad32x16::execute(taddr + uint32_t(c * 16), v);
                    rz::TmemLoadWait::execute(v);
                    if (c == 3) {
                        rz::Tcgen05FenceBefore::execute();
                        __syncwarp();
                        if (lane == 0) rz::BarrierArrive::execute(&pipe.tmem_empty[acc]);
                    }
                    rz::ScalePromoteFma::execute(&accum[c * 16], v, s);
                }
                if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
            }
            if (ok && row_ok) {
                __nv_bfloat16* crow = p.C + (long long)row * p.ldc + col0;
#pragma unroll
                for (int c = 0; c < kCols / 8; ++c) {
                    if (col0 + c * 8 < p.N) {
                        float f[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i) f[i] = accum[c * 8 + i];
                        rz::RowStoreVec16::execute(crow + c * 8,
                            rz::BiasActFma::execute(f, p.bias ? p.bias + col0 + c * 8 : nullptr, p.act,
                                    p.c_in ? p.c_in + (long long)row * p.ldcin + col0 + c * 8 : nullptr, p.alpha, p.beta));
                    }
                }
            }
        }
    }
    rz::Tcgen05FenceBefore::execute();
    __syncthreads();
    if (warp == 1) {
        rz::Tcgen05FenceAfter::execute();
        rz::TmemDealloc<1>::execute(tmem_base, kN128TmemCols);
    }
}

template <bool kFp8>
int launch_gemm(const void* A, const void* B, const float* sA, const float* sB, const float* bias, int act, void* C,
                int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb, int64_t ldc, int64_t n_begin, int64_t n_end,
                void* stream, uint32_t* status_dev, const void* c_in = nullptr, int64_t ldcin = 0, float alpha = 1.0f,
                float beta = 0.0f, float* q_scales = nullptr) {
    using namespace axp_shim;
    constexpr int kElem = kFp8 ? 1 : 2;
    // q_scales non-null (E4M3 block-scaled only): the quantising epilogue - C is then E4M3 bytes [M,N] with ldc bytes per row
    // and q_scales [M, N/128] fp32
    if (q_scales && (!kFp8 || N % 128 != 0 || (n_end - n_begin) % 128 != 0 || ldc % 16 != 0))
        return fail(AXP_ERR_BAD_ARG, "gemm fp8, quantised output: N and the column range must be multiples of the 128-wide scale block, ldq of 16");
    if (c_in && (ldcin < N || ldcin % 8 != 0 || !aligned16(c_in)))
        return fail(AXP_ERR_BAD_ARG, "gemm lincomb: C input needs ldc >= N, a multiple of 8, and a 16-byte aligned base");
    constexpr int kElemsPerRow = kRowBytes / kElem;
    if (!A || !B || !C || (kFp8 && (!sA || !sB))) return fail(AXP_ERR_BAD_ARG, "gemm: null pointer argument");
    if (M <= 0 || N <= 0 || K <= 0) return fail(AXP_ERR_BAD_ARG, "gemm: M, N, K must be positive");
    if (act != AXP_ACT_NONE && act != AXP_ACT_SILU) return fail(AXP_ERR_BAD_ARG, "gemm: unknown activation %d", act);
    if (bias && (reinterpret_cast<uintptr_t>(bias) & 15u)) return fail(AXP_ERR_BAD_ARG, "gemm: bias must be 16-byte aligned");
    if (bias && n_begin % 8 != 0) return fail(AXP_ERR_BAD_ARG, "gemm: n_begin must be a multiple of 8 with a bias");
    if (n_begin < 0 || n_end > N || n_begin > n_end)
        return fail(AXP_ERR_BAD_ARG, "gemm: column range [%lld,%lld) outside [0,%lld)", (long long)n_begin,
                    (long long)n_end, (long long)N);
    if (M > INT32_MAX || N > INT32_MAX || K > INT32_MAX) return fail(AXP_ERR_UNSUPPORTED, "gemm: extent above 2^31-1");
    if (kFp8) {
        if (K % 128 != 0) return fail(AXP_ERR_BAD_ARG, "gemm fp8: K=%lld is not a multiple of the 128-wide scale block", (long long)K);
        if (n_begin % 128 != 0) return fail(AXP_ERR_BAD_ARG, "gemm fp8: n_begin=%lld is not a multiple of 128", (long long)n_begin);
        if (lda % 16 != 0 || ldb % 16 != 0) return fail(AXP_ERR_BAD_ARG, "gemm fp8: lda/ldb must be multiples of 16 elements");
    } else {
        if (K % 8 != 0 || lda % 8 != 0 || ldb % 8 != 0 || n_begin % 8 != 0)
            return fail(AXP_ERR_BAD_ARG, "gemm bf16: K, lda, ldb and n_begin must be multiples of 8 elements");
    }
    // the epilogues write (and read bias / C input) eight columns at a time
    if ((n_end - n_begin) % 8 != 0)
        return fail(AXP_ERR_BAD_ARG, "gemm: the column range [%lld,%lld) must span a multiple of 8 columns", (long long)n_begin, (long long)n_end);
    if (lda < K || ldb < K || ldc < N) return fail(AXP_ERR_BAD_ARG, "gemm: leading dimension smaller than the row length");
    if (ldc % 8 != 0) return fail(AXP_ERR_BAD_ARG, "gemm: ldc must be a multiple of 8 elements");
    if (!aligned16(A) || !aligned16(B) || !aligned16(C)) return fail(AXP_ERR_BAD_ARG, "gemm: base pointers must be 16-byte aligned");
    if (n_begin == n_end) return AXP_OK;

    DeviceInfo dev;
    if (int rc = current_device_info(&dev); rc != AXP_OK) return rc;

    // tuning options (axp_sm100_set_option): epilogue warpgroups and CTAs per MMA
    const int epi_wg_opt = axp_shim::option_slot(axp_shim::kOptGemmEpiWg).load(std::memory_order_relaxed);
    const int cta_group_opt = axp_shim::option_slot(axp_shim::kOptGemmCtaGroup).load(std::memory_order_relaxed);
    // defaults (measured on B200): CTA pairs for both; FP8 block-scaled = two epilogue warpgroups (a thread carries the
    // 128 running sums of its row), BF16 = four.  (With a releasing remote arrive for the per-K-block accumulator
    // hand-over the FP8 pair was 45 % slower than single CTAs; with the relaxed arrive it is 3 % faster: 2115 against
    // 2053 TFLOP/s on 8192^3.)
    constexpr cfg::Gemm kDefault = kFp8 ? cfg::kGemmFp8 : cfg::kGemmBf16;
    // (the quantising epilogue needs a thread to own a whole 128-column scale block: two epilogue warpgroups)
    const int epi_wg = q_scales ? 2 : (epi_wg_opt == 2 || epi_wg_opt == 4) ? epi_wg_opt : kDefault.threads / 128 - 1;
    const int cta_group = (cta_group_opt == 1 || cta_group_opt == 2) ? cta_group_opt : kDefault.cta_group;
    const int b_box_div = cta_group;      // a CTA of a pair loads half of the tile's B rows

    const int64_t n_local = n_end - n_begin;
    const uint8_t* b_base = static_cast<const uint8_t*>(B) + n_begin * ldb * kElem;
    const CUtensorMapDataType dt = kFp8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    CUtensorMap tmA, tmB;
    {
        const uint64_t dims[2] = {uint64_t(K), uint64_t(M)};
        const uint64_t strides[1] = {uint64_t(lda) * kElem};
        const uint32_t box[2] = {uint32_t(kElemsPerRow), uint32_t(kBM)};
        if (int rc = make_tensor_map(&tmA, dt, 2, A, dims, strides, box); rc != AXP_OK) return rc;
    }
    {
        const uint64_t dims[2] = {uint64_t(K), uint64_t(n_local)};
        const uint64_t strides[1] = {uint64_t(ldb) * kElem};
        const uint32_t box[2] = {uint32_t(kElemsPerRow), uint32_t(kBN / b_box_div)};
        if (int rc = make_tensor_map(&tmB, dt, 2, b_base, dims, strides, box); rc != AXP_OK) return rc;
    }

    GemmParams p = {};
    p.sA = sA;
    p.sB = sB;
    p.C = static_cast<__nv_bfloat16*>(C) + n_begin;
    p.M = int(M);
    p.N = int(n_local);
    p.k_blocks = int((K + kElemsPerRow - 1) / kElemsPerRow);
    p.scale_ld = int(K / 128);
    p.sb_row0 = int(n_begin / 128);
    p.bias = bias ? bias + n_begin : nullptr;
    p.act = act;
    p.c_in = c_in ? static_cast<const __nv_bfloat16*>(c_in) + n_begin : nullptr;
    p.ldcin = ldcin;
    p.alpha = alpha;
    p.beta = beta;
    p.ldc = ldc;
    p.status = status_dev;
    if (q_scales) {
        p.C = nullptr;
        p.q_out = static_cast<uint8_t*>(C) + n_begin;
        p.q_scales = q_scales + n_begin / 128;
        p.ldq = ldc;
        p.q_scale_ld = int(N / 128);
    }
#if defined(AXP_SM100_LATENCY_PROBES)
    p.debug = reinterpret_cast<unsigned long long*>(axp_shim::debug_pointer().load(std::memory_order_relaxed));
    p.experiment = axp_shim::option_slot(axp_shim::kOptGemmExperiment).load(std::memory_order_relaxed);
#endif

    const int64_t tile_m = kBM * cta_group;
    const int64_t tiles = ((M + tile_m - 1) / tile_m) * ((n_local + kBN - 1) / kBN);
    const int64_t slots = dev.sm_count / cta_group;
    const int grid = int(tiles < slots ? tiles : slots) * cta_group;
    static thread_local int attr_set_for_device[2][4] = {{-1, -1, -1, -1}, {-1, -1, -1, -1}};
    auto launch = [&](auto kernel, int threads, int smem_bytes, int slot) -> int {
        if (attr_set_for_device[kFp8][slot] != dev.device) {
            const int need = threads == 384 ? 128 * 40 + 256 * 232 : 128 * 32 + 512 * 112;
            if (int rc = check_register_pool(kernel, threads, need, "gemm"); rc != AXP_OK) return rc;
            AXP_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
            attr_set_for_device[kFp8][slot] = dev.device;
        }
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(unsigned(grid), 1, 1);
        cfg.blockDim = dim3(unsigned(threads), 1, 1);
        cfg.dynamicSmemBytes = size_t(smem_bytes);
        cfg.stream = static_cast<cudaStream_t>(stream);
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = unsigned(cta_group);
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        AXP_CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, tmA, tmB, tmB, p));
        return AXP_OK;
    };
    if constexpr (kFp8) {
        // tuning option "gemm.fp8_tile": 0 = library default, 128 = 128 x 128 tiles with two CTAs per SM, 256 = 128 x 256 tiles
        const int tile_opt = option_slot(kOptGemmFp8Tile).load(std::memory_order_relaxed);
        const int tile_n = (tile_opt == 128 || tile_opt == 256) ? tile_opt : kDefaultFp8TileN;
        if (tile_n == 128 && cta_group_opt == 0 && epi_wg_opt == 0) {
            CUtensorMap tmB128;
            const uint64_t dims[2] = {uint64_t(K), uint64_t(n_local)};
            const uint64_t strides[1] = {uint64_t(ldb)};
            const uint32_t box[2] = {128u, 128u};
            if (int rc = make_tensor_map(&tmB128, dt, 2, b_base, dims, strides, box); rc != AXP_OK) return rc;
            static thread_local int n128_attr_device = -1;
            if (n128_attr_device != dev.device) {
                if (int rc = check_register_pool(gemm_fp8_n128_kernel, 384, 128 * 32 + 256 * 104, "gemm fp8 128x128"); rc != AXP_OK) return rc;
                AXP_CUDA_TRY(cudaFuncSetAttribute(gemm_fp8_n128_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kN128DynSmem));
                n128_attr_device = dev.device;
            }
            const int64_t tiles128 = ((M + kBM - 1) / kBM) * ((n_local + 127) / 128);
            const int64_t slots128 = int64_t(dev.sm_count) * 2;
            const int grid128 = int(tiles128 < slots128 ? tiles128 : slots128);
            gemm_fp8_n128_kernel<<<grid128, 384, kN128DynSmem, static_cast<cudaStream_t>(stream)>>>(tmA, tmB128, p);
            AXP_CUDA_TRY(cudaGetLastError());
            return AXP_OK;
        }
    }
    if (cta_group == 2) {
        if (epi_wg == 4) return launch(gemm_kernel<kFp8, 4, 2>, 640, StageCfg<2>::kDynSmem, 3);
        return launch(gemm_kernel<kFp8, 2, 2>, 384, StageCfg<2>::kDynSmem, 2);
    }
    if (epi_wg == 4) return launch(gemm_kernel<kFp8, 4, 1>, 640, StageCfg<1>::kDynSmem, 1);
    return launch(gemm_kernel<kFp8, 2, 1>, 384, StageCfg<1>::kDynSmem, 0);
}

// X [M,K], Wg / Wu [N,K] bf16 -> H[:, n_begin:n_end) = bf16( SiLU(X.Wg^T) * (X.Wu^T) )
int launch_gated(const void* X, const void* Wg, const void* Wu, void* H, int64_t M, int64_t N, int64_t K, int64_t ldx,
                 int64_t ldwg, int64_t ldwu, int64_t ldh, int64_t n_begin, int64_t n_end, void* stream, uint32_t* status_dev) {
    using namespace axp_shim;
    if (!X || !Wg || !Wu || !H) return fail(AXP_ERR_BAD_ARG, "gemm swiglu: null pointer argument");
    if (M <= 0 || N <= 0 || K <= 0) return fail(AXP_ERR_BAD_ARG, "gemm swiglu: M, N, K must be positive");
    if (n_begin < 0 || n_end > N || n_begin > n_end)
        return fail(AXP_ERR_BAD_ARG, "gemm swiglu: column range [%lld,%lld) outside [0,%lld)", (long long)n_begin, (long long)n_end, (long long)N);
    if (M > INT32_MAX || N > INT32_MAX || K > INT32_MAX) return fail(AXP_ERR_UNSUPPORTED, "gemm swiglu: extent above 2^31-1");
    if (K % 8 != 0 || ldx % 8 != 0 || ldwg % 8 != 0 || ldwu % 8 != 0 || ldh % 8 != 0 || n_begin % 8 != 0)
        return fail(AXP_ERR_BAD_ARG, "gemm swiglu: K, leading dimensions and n_begin must be multiples of 8 elements");
    if ((n_end - n_begin) % 8 != 0)
        return fail(AXP_ERR_BAD_ARG, "gemm swiglu: the column range [%lld,%lld) must span a multiple of 8 columns", (long long)n_begin, (long long)n_end);
    if (ldx < K || ldwg < K || ldwu < K || ldh < N) return fail(AXP_ERR_BAD_ARG, "gemm swiglu: leading dimension smaller than the row length");
    if (!aligned16(X) || !aligned16(Wg) || !aligned16(Wu) || !aligned16(H)) return fail(AXP_ERR_BAD_ARG, "gemm swiglu: base pointers must be 16-byte aligned");
    if (n_begin == n_end) return AXP_OK;
    DeviceInfo dev;
    if (int rc = current_device_info(&dev); rc != AXP_OK) return rc;
    const int cta_group_opt = option_slot(kOptGemmCtaGroup).load(std::memory_order_relaxed);
    const int cta_group = (cta_group_opt == 1 || cta_group_opt == 2) ? cta_group_opt : 2;
    const int64_t n_local = n_end - n_begin;
    CUtensorMap tmA, tmG, tmU;
    {
        const uint64_t dims[2] = {uint64_t(K), uint64_t(M)};
        const uint64_t strides[1] = {uint64_t(ldx) * 2};
        const uint32_t box[2] = {64u, uint32_t(kBM)};
        if (int rc = make_tensor_map(&tmA, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, X, dims, strides, box); rc != AXP_OK) return rc;
    }
    {
        const uint64_t dims[2] = {uint64_t(K), uint64_t(n_local)};
        const uint32_t box[2] = {64u, uint32_t(kBN / 2)};
        const uint64_t sg[1] = {uint64_t(ldwg) * 2}, su[1] = {uint64_t(ldwu) * 2};
        const uint8_t* g0 = static_cast<const uint8_t*>(Wg) + n_begin * ldwg * 2;
        const uint8_t* u0 = static_cast<const uint8_t*>(Wu) + n_begin * ldwu * 2;
        if (int rc = make_tensor_map(&tmG, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, g0, dims, sg, box); rc != AXP_OK) return rc;
        if (int rc = make_tensor_map(&tmU, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, u0, dims, su, box); rc != AXP_OK) return rc;
    }
    GemmParams p = {};
    p.C = static_cast<__nv_bfloat16*>(H) + n_begin;
    p.M = int(M);
    p.N = int(n_local);
    p.k_blocks = int((K + 63) / 64);
    p.ldc = ldh;
    p.status = status_dev;
    const int64_t tile_m = kBM * cta_group;
    const int64_t tiles = ((M + tile_m - 1) / tile_m) * ((n_local + kBN / 2 - 1) / (kBN / 2));
    const int64_t slots = dev.sm_count / cta_group;
    const int grid = int(tiles < slots ? tiles : slots) * cta_group;
    static thread_local int attr_set_for_device[2] = {-1, -1};
    auto launch = [&](auto kernel, int smem_bytes, int slot) -> int {
        if (attr_set_for_device[slot] != dev.device) {
            if (int rc = check_register_pool(kernel, 640, 128 * 32 + 512 * 112, "gemm swiglu"); rc != AXP_OK) return rc;
            AXP_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
            attr_set_for_device[slot] = dev.device;
        }
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(unsigned(grid), 1, 1);
        cfg.blockDim = dim3(640, 1, 1);
        cfg.dynamicSmemBytes = size_t(smem_bytes);
        cfg.stream = static_cast<cudaStream_t>(stream);
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = unsigned(cta_group);
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        AXP_CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, tmA, tmG, tmU, p));
        return AXP_OK;
    };
    if (cta_group == 2) return launch(gemm_kernel<false, 4, 2, true>, StageCfg<2>::kDynSmem, 1);
    return launch(gemm_kernel<false, 4, 1, true>, StageCfg<1>::kDynSmem, 0);
}

// E4M3 block-scaled operands: X [M,K] with 1x128 scales sX, Wg / Wu [N,K] with 128x128 scales sWg / sWu
// `Hq_scales` non-null: the quantising epilogue - H is then E4M3 bytes [M,N] (ldh in bytes = elements) and Hq_scales
// [M, N/128] fp32, the operand pair of the next block-scaled GEMM
int launch_gated_fp8(const void* X, const void* Wg, const void* Wu, const float* sX, const float* sWg, const float* sWu, void* H, int64_t M,
                     int64_t N, int64_t K, int64_t ldx, int64_t ldwg, int64_t ldwu, int64_t ldh, int64_t n_begin, int64_t n_end, void* stream,
                     uint32_t* status_dev, float* Hq_scales = nullptr) {
    using namespace axp_shim;
    if (!X || !Wg || !Wu || !H || !sX || !sWg || !sWu) return fail(AXP_ERR_BAD_ARG, "gemm fp8 swiglu: null pointer argument");
    if (Hq_scales && (N % 128 != 0 || (n_end - n_begin) % 128 != 0 || ldh % 16 != 0))
        return fail(AXP_ERR_BAD_ARG, "gemm fp8 swiglu, quantised output: N and the column range must be multiples of the 128-wide scale block, ldq of 16");
    if (M <= 0 || N <= 0 || K <= 0) return fail(AXP_ERR_BAD_ARG, "gemm fp8 swiglu: M, N, K must be positive");
    if (n_begin < 0 || n_end > N || n_begin > n_end)
        return fail(AXP_ERR_BAD_ARG, "gemm fp8 swiglu: column range [%lld,%lld) outside [0,%lld)", (long long)n_begin, (long long)n_end, (long long)N);
    if (M > INT32_MAX || N > INT32_MAX || K > INT32_MAX) return fail(AXP_ERR_UNSUPPORTED, "gemm fp8 swiglu: extent above 2^31-1");
    if (K % 128 != 0) return fail(AXP_ERR_BAD_ARG, "gemm fp8 swiglu: K=%lld is not a multiple of the 128-wide scale block", (long long)K);
    if (n_begin % 128 != 0) return fail(AXP_ERR_BAD_ARG, "gemm fp8 swiglu: n_begin=%lld is not a multiple of 128", (long long)n_begin);
    if (ldx % 16 != 0 || ldwg % 16 != 0 || ldwu % 16 != 0 || ldh % 8 != 0)
        return fail(AXP_ERR_BAD_ARG, "gemm fp8 swiglu: operand leading dimensions must be multiples of 16, ldh of 8 elements");
    if ((n_end - n_begin) % 8 != 0)
        return fail(AXP_ERR_BAD_ARG, "gemm fp8 swiglu: the column range [%lld,%lld) must span a multiple of 8 columns", (long long)n_begin, (long long)n_end);
    if (ldx < K || ldwg < K || ldwu < K || ldh < N) return fail(AXP_ERR_BAD_ARG, "gemm fp8 swiglu: leading dimension smaller than the row length");
    if (!aligned16(X) || !aligned16(Wg) || !aligned16(Wu) || !aligned16(H)) return fail(AXP_ERR_BAD_ARG, "gemm fp8 swiglu: base pointers must be 16-byte aligned");
    if (n_begin == n_end) return AXP_OK;
    DeviceInfo dev;
    if (int rc = current_device_info(&dev); rc != AXP_OK) return rc;
    const int64_t n_local = n_end - n_begin;
    CUtensorMap tmA, tmG, tmU;
    {
        const uint64_t dims[2] = {uint64_t(K), uint64_t(M)};
        const uint64_t strides[1] = {uint64_t(ldx)};
        const uint32_t box[2] = {128u, uint32_t(kBM)};
        if (int rc = make_tensor_map(&tmA, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, X, dims, strides, box); rc != AXP_OK) return rc;
    }
    {
        const uint64_t dims[2] = {uint64_t(K), uint64_t(n_local)};
        const uint32_t box[2] = {128u, uint32_t(kBN / 2)};
        const uint64_t sg[1] = {uint64_t(ldwg)}, su[1] = {uint64_t(ldwu)};
        const uint8_t* g0 = static_cast<const uint8_t*>(Wg) + n_begin * ldwg;
        const uint8_t* u0 = static_cast<const uint8_t*>(Wu) + n_begin * ldwu;
        if (int rc = make_tensor_map(&tmG, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, g0, dims, sg, box); rc != AXP_OK) return rc;
        if (int rc = make_tensor_map(&tmU, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, u0, dims, su, box); rc != AXP_OK) return rc;
    }
    GemmParams p = {};
    p.sA = sX;
    p.sB = sWg;
    p.sB2 = sWu;
    p.C = static_cast<__nv_bfloat16*>(H) + n_begin;
    p.M = int(M);
    p.N = int(n_local);
    p.k_blocks = int(K / 128);
    p.scale_ld = int(K / 128);
    p.sb_row0 = int(n_begin / 128);
    p.alpha = 1.0f;
    p.ldc = ldh;
    p.status = status_dev;
    if (Hq_scales) {
        p.C = nullptr;
        p.q_out = static_cast<uint8_t*>(H) + n_begin;
        p.q_scales = Hq_scales + n_begin / 128;
        p.ldq = ldh;
        p.q_scale_ld = int(N / 128);
    }
    // Single CTAs by default: with two scale streams per K block the pair form (the leader stages the gate rows, its peer
    // the up rows; option "gemm.cta_group" = 2) measured slower here (1681 against 1826 TFLOP/s on the MLP gate / up shape),
    // unlike the plain block-scaled kernel.
    const int cta_group = option_slot(kOptGemmCtaGroup).load(std::memory_order_relaxed) == 2 ? 2 : 1;
    const int64_t tile_m = kBM * cta_group;
    const int64_t tiles = ((M + tile_m - 1) / tile_m) * ((n_local + kBN / 2 - 1) / (kBN / 2));
    const int64_t slots = dev.sm_count / cta_group;
    const int grid = int(tiles < slots ? tiles : slots) * cta_group;
    static thread_local int attr_set_for_device[2] = {-1, -1};
    auto launch = [&](auto kernel, int smem_bytes, int slot) -> int {
        if (attr_set_for_device[slot] != dev.device) {
            if (int rc = check_register_pool(kernel, 384, 128 * 40 + 256 * 232, "gemm fp8 swiglu"); rc != AXP_OK) return rc;
            AXP_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
            attr_set_for_device[slot] = dev.device;
        }
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(unsigned(grid), 1, 1);
        cfg.blockDim = dim3(384, 1, 1);
        cfg.dynamicSmemBytes = size_t(smem_bytes);
        cfg.stream = static_cast<cudaStream_t>(stream);
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = unsigned(cta_group);
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        AXP_CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, tmA, tmG, tmU, p));
        return AXP_OK;
    };
    if (cta_group == 2) return launch(gemm_kernel<true, 2, 2, true>, StageCfg<2>::kDynSmem, 1);
    return launch(gemm_kernel<true, 2, 1, true>, StageCfg<1>::kDynSmem, 0);
}

}  // namespace

extern "C" int axp_sm100_gemm_fp8_blockscaled_swiglu(const void* X, const void* Wg, const void* Wu, const float* sX, const float* sWg,
                                                     const float* sWu, void* H, int64_t M, int64_t N, int64_t K, int64_t ldx,
                                                     int64_t ldwg, int64_t ldwu, int64_t ldh, int64_t n_begin, int64_t n_end,
                                                     void* stream, uint32_t* status_dev) {
    axp_shim::NvtxRange nvtx_range("axp_sm100_gemm_fp8_blockscaled_swiglu");
    return launch_gated_fp8(X, Wg, Wu, sX, sWg, sWu, H, M, N, K, ldx, ldwg, ldwu, ldh, n_begin, n_end, stream, status_dev);
}

extern "C" int axp_sm100_gemm_fp8_blockscaled_swiglu_quant(const void* X, const void* Wg, const void* Wu, const float* sX, const float* sWg,
                                                           const float* sWu, void* Hq, float* Hq_scales, int64_t M, int64_t N, int64_t K,
                                                           int64_t ldx, int64_t ldwg, int64_t ldwu, int64_t ldq, int64_t n_begin,
                                                           int64_t n_end, void* stream, uint32_t* status_dev) {
    axp_shim::NvtxRange nvtx_range("axp_sm100_gemm_fp8_blockscaled_swiglu_quant");
    if (!Hq_scales) return axp_shim::fail(AXP_ERR_BAD_ARG, "gemm fp8 swiglu, quantised output: scales pointer is null");
    return launch_gated_fp8(X, Wg, Wu, sX, sWg, sWu, Hq, M, N, K, ldx, ldwg, ldwu, ldq, n_begin, n_end, stream, status_dev, Hq_scales);
}

extern "C" int axp_sm100_gemm_bf16_swiglu(const void* X, const void* Wg, const void* Wu, void* H, int64_t M, int64_t N,
                                          int64_t K, int64_t ldx, int64_t ldwg, int64_t ldwu, int64_t ldh,
                                          int64_t n_begin, int64_t n_end, void* stream, uint32_t* status_dev) {
    axp_shim::NvtxRange nvtx_range("axp_sm100_gemm_bf16_swiglu");
    return launch_gated(X, Wg, Wu, H, M, N, K, ldx, ldwg, ldwu, ldh, n_begin, n_end, stream, status_dev);
}

extern "C" int axp_sm100_gemm_fp8_blockscaled(const void* A, const void* B, const float* sA, const float* sB, void* C,
                                              int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb, int64_t ldc,
                                              int64_t n_begin, int64_t n_end, void* stream, uint32_t* status_dev) {
    axp_shim::NvtxRange nvtx_range("axp_sm100_gemm_fp8_blockscaled");
    return launch_gemm<true>(A, B, sA, sB, nullptr, AXP_ACT_NONE, C, M, N, K, lda, ldb, ldc, n_begin, n_end, stream, status_dev);
}

extern "C" int axp_sm100_gemm_fp8_blockscaled_quant(const void* A, const void* B, const float* sA, const float* sB, const float* bias,
                                                    int act, void* Cq, float* Cq_scales, int64_t M, int64_t N, int64_t K, int64_t lda,
                                                    int64_t ldb, int64_t ldq, int64_t n_begin, int64_t n_end, void* stream,
                                                    uint32_t* status_dev) {
    axp_shim::NvtxRange nvtx_range("axp_sm100_gemm_fp8_blockscaled_quant");
    if (!Cq_scales) return axp_shim::fail(AXP_ERR_BAD_ARG, "gemm fp8, quantised output: scales pointer is null");
    return launch_gemm<true>(A, B, sA, sB, bias, act, Cq, M, N, K, lda, ldb, ldq, n_begin, n_end, stream, status_dev, nullptr, 0, 1.0f, 0.0f,
                             Cq_scales);
}

extern "C" int axp_sm100_gemm_bf16_lincomb(const void* A, const void* B, const void* Cin, void* D, float alpha, float beta, int64_t M,
                                           int64_t N, int64_t K, int64_t lda, int64_t ldb, int64_t ldcin, int64_t ldd,
                                           int64_t n_begin, int64_t n_end, void* stream, uint32_t* status_dev) {
    axp_shim::NvtxRange nvtx_range("axp_sm100_gemm_bf16_lincomb");
    if (!Cin) return axp_shim::fail(AXP_ERR_BAD_ARG, "gemm lincomb: C input is null");
    return launch_gemm<false>(A, B, nullptr, nullptr, nullptr, AXP_ACT_NONE, D, M, N, K, lda, ldb, ldd, n_begin, n_end, stream, status_dev,
                              Cin, ldcin, alpha, beta);
}

extern "C" int axp_sm100_gemm_fp8_blockscaled_lincomb(const void* A, const void* B, const float* sA, const float* sB, const void* Cin,
                                                      void* D, float alpha, float beta, int64_t M, int64_t N, int64_t K, int64_t lda,
                                                      int64_t ldb, int64_t ldcin, int64_t ldd, int64_t n_begin, int64_t n_end,
                                                      void* stream, uint32_t* status_dev) {
    axp_shim::NvtxRange nvtx_range("axp_sm100_gemm_fp8_blockscaled_lincomb");
    if (!Cin) return axp_shim::fail(AXP_ERR_BAD_ARG, "gemm lincomb: C input is null");
    return launch_gemm<true>(A, B, sA, sB, nullptr, AXP_ACT_NONE, D, M, N, K, lda, ldb, ldd, n_begin, n_end, stream, status_dev, Cin,
                             ldcin, alpha, beta);
}

extern "C" int axp_sm100_gemm_fp8_blockscaled_bias_act(const void* A, const void* B, const float* sA, const float* sB,
                                                       const float* bias, void* C, int64_t M, int64_t N, int64_t K,
                                                       int64_t lda, int64_t ldb, int64_t ldc, int64_t n_begin,
                                                       int64_t n_end, int act, void* stream, uint32_t* status_dev) {
    axp_shim::NvtxRange nvtx_range("axp_sm100_gemm_fp8_blockscaled_bias_act");
    if (!bias) return axp_shim::fail(AXP_ERR_BAD_ARG, "gemm bias_act: bias is null");
    return launch_gemm<true>(A, B, sA, sB, bias, act, C, M, N, K, lda, ldb, ldc, n_begin, n_end, stream, status_dev);
}

extern "C" int axp_sm100_gemm_bf16(const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K,
                                   int64_t lda, int64_t ldb, int64_t ldc, int64_t n_begin, int64_t n_end,
                                   void* stream, uint32_t* status_dev) {
    axp_shim::NvtxRange nvtx_range("axp_sm100_gemm_bf16");
    return launch_gemm<false>(A, B, nullptr, nullptr, nullptr, AXP_ACT_NONE, C, M, N, K, lda, ldb, ldc, n_begin, n_end, stream,
                              status_dev);
}

extern "C" int axp_sm100_gemm_bf16_bias_act(const void* A, const void* B, const float* bias, void* C, int64_t M, int64_t N,
                                            int64_t K, int64_t lda, int64_t ldb, int64_t ldc, int64_t n_begin,
                                            int64_t n_end, int act, void* stream, uint32_t* status_dev) {
    axp_shim::NvtxRange nvtx_range("axp_sm100_gemm_bf16_bias_act");
    if (!bias) return axp_shim::fail(AXP_ERR_BAD_ARG, "gemm bias_act: bias is null");
    return launch_gemm<false>(A, B, nullptr, nullptr, bias, act, C, M, N, K, lda, ldb, ldc, n_begin, n_end, stream, status_dev);
}
