// sm_100a flash-attention forward kernels behind axp_sm100_attn_fwd_bf16 /
// axp_sm100_attn_fwd_fp8.
//
// Recipe realised (reference include/axp/level3/recipes/attention/process.hpp:1766-1864):
// per (Q tile, KV tile) step  S = Q.K^T -> mask -> softmax state update -> P cast ->
// O += P.V, with the softmax state (m,l) kept per query row (the reference's
// tile-wide reduction is not reproduced) and the accumulator normalised once at
// the end instead of after every tile.  Softmax scale, LSE output, GQA head
// mapping and the FP8 descales are additions of the benchmark configurations.
//
// One CTA owns 256 query rows of one (batch, head): two 128-row Q tiles that
// share every K/V tile brought into shared memory.  384 threads:
//   warps 0-3   softmax / correction / epilogue for Q tile 0 (thread = query row)
//   warps 4-7   the same for Q tile 1
//   warp  8     TMA producer (Q once, then K_j, V_j through a small ring)
//   warp  9     tcgen05.mma issuer (both Q tiles, or Q tile 0 when warp 10 issues for
//               Q tile 1); owns the TMEM allocation
// Tensor memory (512 columns): S0 [0,128) S1 [128,256) O0 [256,384) O1 [384,512), fp32.
// V is the B operand of P.V in its natural [key][d] layout (MN-major descriptor).
// The softmax of a Q tile, its Q.K^T and its P.V form a dependent chain; three
// arrangements keep the tensor core and the softmax busy at the same time:
//   * 128-key tiles, P over the first columns of S in tensor memory (A operand of P.V
//     from tensor memory): MMA order S0 S1 | PV0 S0' PV1 S1' | ..., one Q tile's MMAs
//     run while the other tile's softmax runs;
//   * bf16 default: 64-key tiles, two 64-column S buffers per Q tile, so the Q.K^T of
//     step j + 2 follows the P.V of step j and the softmax never waits for scores;
//     one issuing thread per Q tile, because a tcgen05.mma costs its issuing thread
//     about 50 cycles and the 64-key MMAs are shorter than that;
//   * E4M3 default: 128-key tiles, P through shared memory (K-major, swizzled, two
//     buffers per Q tile), so S is free once the softmax holds it in registers and the
//     next Q.K^T is issued while the exponentials run.
// The accumulator is only rescaled when a row maximum grows by more than 2^8
// (the stale maximum is used consistently for P, l and O, so the result is
// unchanged); otherwise O stays untouched in tensor memory between P.V steps.
#include <cuda_bf16.h>

#include <atomic>

#include "axp/realize/sm100.hpp"
#include "axp/realize/sm100_mask.hpp"
#include "host_common.hpp"
#include "kernel_config.hpp"

namespace rz = axp::realize::sm100;

namespace {

constexpr int kTileM = 128;   // query rows per Q tile
constexpr int kHeadDim = 128;
constexpr int kQTiles = 2;    // Q tiles per CTA
constexpr int kAttnThreads = 384;
constexpr int kMaxKvStages = 4;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr float kRescaleThreshold = 8.0f;   // log2 units
constexpr float kDefaultRescaleFp8 = 8.0f;  // E4M3 prefill kernels (0 = standard online softmax)
constexpr int kDefaultExpModeBf16 = 1;   // measured on cfg3 (64-key tiles, two issuers): 2/8 983, SFU only 970 TFLOP/s
constexpr int kDefaultExpModeFp8 = 1;    // measured on cfg4: 2/8 1281, SFU only 1256, 3/8 1273, 4/8 1272 TFLOP/s
constexpr bool kDefaultPSmemFp8 = true;
constexpr int kDefaultKvTileBf16 = 64;

// kPSmem: P goes to the P.V MMA through shared memory (K-major, 128-byte swizzle, two buffers per Q tile) instead of
// overwriting its S region in tensor memory.  S is then free as soon as the softmax has read it, so the next
// Q.K^T of the same Q tile is issued while the exponentials of this one still run.
// kN: keys per KV tile.  With kN = 64 (bf16) each Q tile owns two 64-column S buffers in tensor memory, so the
// Q.K^T of step j + 2 is issued right after the P.V of step j and the softmax of a Q tile never waits for the
// tensor core (with kN = 128 the single S buffer makes Q.K^T, softmax and P.V of a Q tile one serial chain).
template <bool kFp8, bool kPSmem = false, int kN = 128>
struct AttnCfg {
    static constexpr int kElem = kFp8 ? 1 : 2;
    static constexpr int kSub = kFp8 ? 1 : 2;                     // 128-byte spans per row of D
    static constexpr int kSubCols = 128 / kElem;                   // elements per span
    static constexpr int kSubBytes = 128 * 128;                    // one [128 rows x 128 B] sub-tile
    static constexpr int kTileBytes = kSub * kSubBytes;            // Q tile (and a P tile in shared memory)
    static constexpr int kKvSubBytes = kN * 128;                   // one [kN keys x 128 B] sub-tile
    static constexpr int kKvTileBytes = kSub * kKvSubBytes;        // K or V tile
    static constexpr int kSBufs = 128 / kN;                        // S buffers per Q tile (each kN columns)
    static constexpr int kKvStages = kFp8 ? (kPSmem ? 3 : 4) : (kN == 64 ? 4 : 2);
    static constexpr int kPTiles = kPSmem ? 2 * kQTiles : 0;
    static constexpr int kMmaK = 32 / kElem;                       // elements of K per MMA
    static constexpr int kSteps = 128 / kMmaK;                     // MMAs per Q.K^T (contraction over the head dimension)
    static constexpr int kPvSteps = kN / kMmaK;                    // MMAs per P.V (contraction over the keys of the tile)
    static constexpr int kSmem = (kQTiles + kPTiles) * kTileBytes + 2 * kKvStages * kKvTileBytes + 1024;
    static_assert(kN == 128 || (kN == 64 && !kFp8 && !kPSmem), "64-key tiles are realised for bf16 with P in tensor memory");
    static_assert(kSmem <= 227 * 1024, "shared memory budget");
};

// the default dispatch (launch_attn) and the configuration header agree
namespace cfg = axp_shim::cfg;
using DefaultCfgBf16 = AttnCfg<false, cfg::kAttnBf16.p_through_smem, cfg::kAttnBf16.kv_tile>;
using DefaultCfgFp8 = AttnCfg<true, cfg::kAttnFp8.p_through_smem, cfg::kAttnFp8.kv_tile>;
static_assert(cfg::kAttnBf16.kv_tile == kDefaultKvTileBf16 && cfg::kAttnFp8.p_through_smem == kDefaultPSmemFp8);
static_assert(cfg::kAttnBf16.kv_stages == DefaultCfgBf16::kKvStages && cfg::kAttnBf16.dyn_smem == DefaultCfgBf16::kSmem);
static_assert(cfg::kAttnFp8.kv_stages == DefaultCfgFp8::kKvStages && cfg::kAttnFp8.dyn_smem == DefaultCfgFp8::kSmem);
static_assert(cfg::kAttnBf16.threads == kAttnThreads && cfg::kAttnFp8.threads == kAttnThreads && cfg::kAttnBf16.q_tiles == kQTiles &&
              cfg::kAttnBf16.tile_q == kTileM && cfg::kAttnBf16.head_dim == kHeadDim);

struct AttnParams {
    void* O;               // bf16 [BH, S, D]
    float* LSE;            // [BH, S] or null
    const float* dq;       // fp8: [B*Hq]
    const float* dk;       // fp8: [B*Hkv]
    const float* dv;       // fp8: [B*Hkv]
    int Sq;                // query rows per (batch, head) of this launch
    int q_per_head;        // = Sq, or smaller when the query heads of a GQA group are stacked into one launch "head":
                           // row r then is query r % q_per_head of group member r / q_per_head
    int Skv;               // keys per head; under the causal mask query i sees keys <= i + (Skv - Sq)
    int Hq;
    int Hkv;
    int causal;
    int bh_begin;
    int num_q_blocks;      // ceil(S / 256)
    int num_heads;         // (batch, head) pairs of this launch; grid.x = num_q_blocks * num_heads
    float scale;           // softmax scale
    uint32_t* status;
#if defined(AXP_SM100_LATENCY_PROBES)
    unsigned long long* debug;   // timestamp buffer of the latency experiments
    int experiment;              // bits 8..: the CTA that is timed
#endif
    // split-KV: CTA z of gridDim.z visits KV tiles [z * tiles_per_split, (z + 1) * tiles_per_split) and, when
    // splits > 1, leaves its unnormalised accumulator (fp32) and (m * c, l) per row in scratch memory
    float rescale_thr;     // log2 units: the reference maximum of a row advances when a tile maximum exceeds it by more than this
    int splits;
    int partial;           // 1: leave partial results (always when splits > 1; also for one share of a KV-sharded call)
    int causal_off;        // under the causal mask query position i (inside its head) sees local keys <= i + causal_off;
                           // Skv - q_per_head for a whole sequence, smaller (possibly negative) for a later KV shard
    int tiles_per_split;
    float* part_o;         // [splits][heads of this call][Sq][128]
    float2* part_ml;       // [splits][heads of this call][Sq]: (row maximum in log2 units, row sum)
    int two_issuers;             // 1: one MMA-issuing thread per Q tile (warps 9 and 10), 0: one for both (warp 9)
};

struct AttnPipe {
    uint64_t q_full[kQTiles];
    uint64_t k_full[kMaxKvStages];
    uint64_t k_empty[kMaxKvStages];
    uint64_t v_full[kMaxKvStages];
    uint64_t v_empty[kMaxKvStages];
    uint64_t s_full[kQTiles][2];   // S of step j: s_full[qt][j % kSBufs] (phase j / kSBufs)
    uint64_t p_full[kQTiles][2];   // P of step j arrives on p_full[qt][j & 1] (phase j >> 1): with two P buffers the softmax
                                   // may finish step j + 1 before the issuer has looked at step j
    uint64_t o_done[kQTiles][2];   // P.V of step j completes o_done[qt][j & 1] (phase j >> 1)
    uint64_t s_free[kQTiles];      // kPSmem: the softmax has taken S out of tensor memory
    uint64_t dbg_bar;          // latency experiments only
    uint32_t tmem_base;
    uint32_t abort_flag;
};

__device__ __forceinline__ void attn_report(const AttnParams& p, AttnPipe* pipe, uint32_t code) {
    *reinterpret_cast<volatile uint32_t*>(&pipe->abort_flag) = 1u;
    if (p.status) atomicOr(p.status, rz::kStatusError | code);
}

// Latency probes (globaltimer stamps at role hand-over points) exist only in builds with
// -DAXP_SM100_LATENCY_PROBES; the production kernels carry none of it.
__device__ __forceinline__ void attn_stamp(const AttnParams& p, int what, int n) {
#if defined(AXP_SM100_LATENCY_PROBES)
    if (p.debug && blockIdx.x == unsigned(p.experiment >> 8) && n < 32) {      // experiment bits 8..: the CTA that is timed
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        p.debug[what * 32 + n] = t;
        if (what == 0) p.debug[480 + n] = (unsigned long long)clock64();   // SM cycles beside the wall clock
    }
#else
    (void)p; (void)what; (void)n;
#endif
}

#if defined(AXP_SM100_LATENCY_PROBES)
constexpr bool kAttnProbes = true;    // p.experiment bits switch parts of the softmax off (results invalid; times only)
#else
constexpr bool kAttnProbes = false;
#endif

// number of KV tiles Q tile `qt` (rows [q0, q0+128)) has to visit
__device__ __forceinline__ int kv_tiles_for(int q0, int Sq, int q_per_head, int Skv, int causal, int causal_off, int tile_n) {
    if (q0 >= Sq) return 0;
    const int all = (Skv + tile_n - 1) / tile_n;
    if (!causal) return all;
    // the last query position (inside its head) among the rows of this Q tile; with stacked heads (q_per_head < Sq,
    // at most 64) every Q tile holds the last query of some head
    const int last_row = (q0 + kTileM - 1 < Sq - 1) ? q0 + kTileM - 1 : Sq - 1;
    const long long last_q = q_per_head < Sq ? q_per_head - 1 : last_row;
    const long long last_k = last_q + causal_off;          // last local key any row of the tile sees
    if (last_k < 0) return 0;                               // the whole KV shard lies in the future of these queries
    const long long n = last_k / tile_n + 1;
    return n < all ? int(n) : all;
}

// kExpMode: 0 = every exponential on the SFU; 1 / 2 / 3 = 2 / 4 / 3 of every 8 pairs as a polynomial on the FMA pipe.
template <bool kFp8, int kExpMode, bool kPSmem, int kN>
__global__ void __launch_bounds__(kAttnThreads, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmO, const AttnParams p) {
    using Cfg = AttnCfg<kFp8, kPSmem, kN>;
    constexpr int kSBufs = Cfg::kSBufs;
    // pairs (of every eight) whose exponentials take the polynomial: none, 2/8, 4/8, 3/8
    constexpr int kPolyMask = kExpMode == 1 ? 0x22 : kExpMode == 2 ? 0xaa : kExpMode == 3 ? 0x4a : 0x00;
    constexpr int kStages = Cfg::kKvStages;
    constexpr uint32_t kFmt = kFp8 ? 0u : 1u;
    constexpr uint32_t kIdescQK = rz::make_instr_desc(kFmt, kFmt, false, false, kTileM, kN);
    constexpr uint32_t kIdescPV = rz::make_instr_desc(kFmt, kFmt, false, true, kTileM, kHeadDim);

    // setmaxnreg only moves registers inside the CTA's launch allocation
    constexpr int kLaunchRegs = (65536 / kAttnThreads) / 8 * 8;      // 168
    constexpr int kProducerRegs = 56, kSoftmaxRegs = 224;
    static_assert(kProducerRegs == cfg::kAttnBf16.producer_regs && kSoftmaxRegs == cfg::kAttnBf16.softmax_regs &&
                  kProducerRegs == cfg::kAttnFp8.producer_regs && kSoftmaxRegs == cfg::kAttnFp8.softmax_regs);
    static_assert(128 * kProducerRegs + 256 * kSoftmaxRegs <= kAttnThreads * kLaunchRegs,
                  "register budgets exceed the CTA's launch allocation");

    extern __shared__ uint8_t dyn_smem_raw[];
    __shared__ AttnPipe pipe;
    if (threadIdx.x == 0) attn_stamp(p, 14, 0);       // kernel entry
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(dyn_smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sQ = smem;
    uint8_t* sK = sQ + kQTiles * Cfg::kTileBytes;
    uint8_t* sV = sK + kStages * Cfg::kKvTileBytes;
    uint8_t* sP = sV + kStages * Cfg::kKvTileBytes;     // kPSmem: [Q tile][buffer] P tiles

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    volatile uint32_t* abort_flag = &pipe.abort_flag;

    // Work order (CTAs start in blockIdx.x order): heads in groups of kHeadGroup; inside a group the heavy (late) query
    // blocks of all its heads come first - under the causal mask their KV range is longest, so the SMs run out of work
    // at about the same time - while the K / V of the group's heads (a few tens of MB) stay in L2.
    constexpr int kHeadGroup = 8;        // measured on the causal bf16 config: 4: 1028, 8: 1079, 16: 1046-1054, 32: 1061 TFLOP/s
    const int group = int(blockIdx.x) / (kHeadGroup * p.num_q_blocks);
    const int in_group = int(blockIdx.x) - group * (kHeadGroup * p.num_q_blocks);
    const int group_heads = p.num_heads - group * kHeadGroup < kHeadGroup ? p.num_heads - group * kHeadGroup : kHeadGroup;
    const int qblk = p.num_q_blocks - 1 - in_group / group_heads;
    const int bh = p.bh_begin + group * kHeadGroup + in_group % group_heads;
    const int batch = bh / p.Hq;
    const int head = bh - batch * p.Hq;
    const int kvh = batch * p.Hkv + head / (p.Hq / p.Hkv);
    const int q_base = qblk * (kQTiles * kTileM);
    // this CTA's share of the KV tiles (all of them unless the call splits the keys)
    const int j_lo = int(blockIdx.z) * p.tiles_per_split;
    auto share = [&](int n_all) {
        const int left = n_all - j_lo;
        return left < 0 ? 0 : (left < p.tiles_per_split ? left : p.tiles_per_split);
    };
    const bool stacked = p.q_per_head < p.Sq;
    const int causal_off = p.causal_off;
    const int n0 = share(kv_tiles_for(q_base, p.Sq, p.q_per_head, p.Skv, p.causal, causal_off, kN));
    const int n1 = share(kv_tiles_for(q_base + kTileM, p.Sq, p.q_per_head, p.Skv, p.causal, causal_off, kN));
    const int n_max = n0 > n1 ? n0 : n1;

    // K_j / V_j of this CTA into ring slot st (the caller has seen the slot free)
    auto load_k = [&](int j, int st) {
        rz::BarrierExpectTx::execute(&pipe.k_full[st], Cfg::kKvTileBytes);
        for (int sub = 0; sub < Cfg::kSub; ++sub)
            rz::BulkTmaCopy3D::execute(&tmK, sK + st * Cfg::kKvTileBytes + sub * Cfg::kKvSubBytes, sub * Cfg::kSubCols, (j_lo + j) * kN, kvh,
                                       &pipe.k_full[st]);
    };
    auto load_v = [&](int j, int st) {
        rz::BarrierExpectTx::execute(&pipe.v_full[st], Cfg::kKvTileBytes);
        for (int sub = 0; sub < Cfg::kSub; ++sub)
            rz::BulkTmaCopy3D::execute(&tmV, sV + st * Cfg::kKvTileBytes + sub * Cfg::kKvSubBytes, sub * Cfg::kSubCols, (j_lo + j) * kN, kvh,
                                       &pipe.v_full[st]);
    };
    const int n_first = n_max < kStages ? n_max : kStages;      // KV tiles whose ring slots are free from the start

    // The producer thread initialises the barriers and at once requests Q and the first ring of K / V tiles: the
    // loads are in flight while tensor memory is allocated and the CTA meets at the first barrier.
    if (warp == 8 && lane == 0) {
        rz::PrefetchTensorMap::execute(&tmQ);
        rz::PrefetchTensorMap::execute(&tmK);
        rz::PrefetchTensorMap::execute(&tmV);
        for (int i = 0; i < kQTiles; ++i) {
            rz::BarrierInit::execute(&pipe.q_full[i], 1);
            rz::BarrierInit::execute(&pipe.s_full[i][0], 1);
            rz::BarrierInit::execute(&pipe.s_full[i][1], 1);
            // softmax hand-overs: one arrival per warp (lane 0 after __syncwarp), not one per thread - 128 arrivals
            // on one shared-memory word serialise
            rz::BarrierInit::execute(&pipe.p_full[i][0], kTileM / 32);
            rz::BarrierInit::execute(&pipe.p_full[i][1], kTileM / 32);
            rz::BarrierInit::execute(&pipe.o_done[i][0], 1);
            rz::BarrierInit::execute(&pipe.o_done[i][1], 1);
            rz::BarrierInit::execute(&pipe.s_free[i], kTileM / 32);
        }
        for (int s = 0; s < kStages; ++s) {
            rz::BarrierInit::execute(&pipe.k_full[s], 1);
            rz::BarrierInit::execute(&pipe.k_empty[s], p.two_issuers ? kQTiles : 1);      // one arrival per issuer
            rz::BarrierInit::execute(&pipe.v_full[s], 1);
            rz::BarrierInit::execute(&pipe.v_empty[s], p.two_issuers ? kQTiles : 1);
        }
        rz::BarrierInit::execute(&pipe.dbg_bar, 1);
        pipe.abort_flag = 0;
        rz::BarrierInitFence::execute();
        for (int qt = 0; qt < kQTiles; ++qt) {
            if ((qt == 0 ? n0 : n1) > 0) {
                rz::BarrierExpectTx::execute(&pipe.q_full[qt], Cfg::kTileBytes);
                for (int sub = 0; sub < Cfg::kSub; ++sub)
                    rz::BulkTmaCopy3D::execute(&tmQ, sQ + qt * Cfg::kTileBytes + sub * Cfg::kSubBytes, sub * Cfg::kSubCols,
                                               q_base + qt * kTileM, bh, &pipe.q_full[qt]);
            }
        }
        for (int j = 0; j < n_first; ++j) {
            load_k(j, j);
            load_v(j, j);
        }
    }
    if (warp == 9) rz::TmemAlloc<1>::execute(&pipe.tmem_base, 512);
    rz::Tcgen05FenceBefore::execute();
    __syncthreads();
    rz::Tcgen05FenceAfter::execute();
    const uint32_t tmem_base = pipe.tmem_base;
    if (threadIdx.x == 0) attn_stamp(p, 14, 1);       // set-up done

    if (warp >= 8) {
        rz::RegDealloc<kProducerRegs>::execute();
        if (warp == 8) {
            // ---------------------------------------------------- TMA producer ----
            // Q and the first n_first KV tiles were requested before the first barrier; the ring goes on from there.
            // The whole warp runs the loop (waits are votes of all lanes); lane 0, which set the barriers up, issues the copies.
            const bool elected = lane == 0;
            int st = n_first == kStages ? 0 : n_first;
            uint32_t phase = n_first == kStages ? 1u : 0u;
            bool ok = true;
            for (int j = n_first; j < n_max && ok; ++j) {
                if (!__all_sync(0xffffffffu, rz::BarrierWait::execute(&pipe.k_empty[st], phase ^ 1u, abort_flag))) {
                    if (elected) attn_report(p, &pipe, rz::kRoleProducer | rz::kBarEmpty);
                    ok = false;
                    break;
                }
                if (elected) load_k(j, st);
                if (!__all_sync(0xffffffffu, rz::BarrierWait::execute(&pipe.v_empty[st], phase ^ 1u, abort_flag))) {
                    if (elected) attn_report(p, &pipe, rz::kRoleProducer | rz::kBarEmpty);
                    ok = false;
                    break;
                }
                if (elected) load_v(j, st);
                if (++st == kStages) { st = 0; phase ^= 1u; }
            }
            // tail: all slots released (every issued MMA has read its operands)
            for (int s = 0; s < kStages && ok; ++s) {
                if (!__all_sync(0xffffffffu, rz::BarrierWait::execute(&pipe.k_empty[st], phase ^ 1u, abort_flag) &&
                                                 rz::BarrierWait::execute(&pipe.v_empty[st], phase ^ 1u, abort_flag))) {
                    if (elected) attn_report(p, &pipe, rz::kRoleProducer | rz::kBarEmpty);
                    ok = false;
                }
                if (++st == kStages) { st = 0; phase ^= 1u; }
            }
        } else if (p.two_issuers && (warp == 9 || warp == 10)) {
            // ------------------------------------- MMA issuers, one per Q tile ----
            // The whole warp runs the loop (every wait is a vote of all lanes, so the lanes stay together) and one
            // elected lane issues: loop control and descriptor arithmetic stay warp-uniform, which makes the issue of a
            // tcgen05.mma about 1.6 times cheaper while the softmax warps compete for the sub-partition's issue slots
            // (micro-benchmark: 58 % against 36 % of the tensor pipe reached by one issuer beside a running softmax).
            const bool leader = rz::elect_one();
            // Each thread follows only its own Q tile's hand-overs; the tensor pipe interleaves the groups in issue
            // order and the issue cost of a tcgen05.mma (about 50 cycles per instruction from one thread) is
            // spread over two threads.  A K / V slot goes back to the producer when both issuers have arrived on
            // its barrier: tcgen05.commit after the last MMA that reads it, or a plain arrive for a KV tile that
            // this Q tile does not visit.
            const int qt = warp - 9;
            const int n = qt == 0 ? n0 : n1;
            const uint32_t tO = tmem_base + uint32_t(256 + qt * 128);
            constexpr uint32_t kTileUnits = Cfg::kTileBytes >> 4;               // descriptor address units are 16 bytes
            constexpr uint32_t kKvTileUnits = Cfg::kKvTileBytes >> 4;
            constexpr uint32_t kSubUnits = Cfg::kSubBytes >> 4;
            constexpr uint32_t kKvSubUnits = Cfg::kKvSubBytes >> 4;
            const uint32_t q_lo = rz::sw128_desc_lo(rz::smem_u32(sQ), 16) + uint32_t(qt) * kTileUnits;
            const uint32_t k_lo = rz::sw128_desc_lo(rz::smem_u32(sK), 16);
            const uint32_t v_lo = rz::sw128_desc_lo(rz::smem_u32(sV), Cfg::kKvSubBytes);
            const uint32_t p_lo = rz::sw128_desc_lo(rz::smem_u32(sP), 16) + uint32_t(qt * 2) * kTileUnits;
            auto issue_qk = [&](int st, int j) {
                if (!leader) return;
                const uint32_t b0 = k_lo + uint32_t(st) * kKvTileUnits;
                const uint32_t d = tmem_base + uint32_t(qt * 128 + (j % kSBufs) * kN);
#pragma unroll
                for (int s = 0; s < Cfg::kSteps; ++s) {
                    const uint32_t in_span = uint32_t(((s * 32) % 128) >> 4);
                    rz::Tcgen05MmaLo<!kFp8>::execute(d, q_lo + uint32_t((s * 32) / 128) * kSubUnits + in_span,
                                                     b0 + uint32_t((s * 32) / 128) * kKvSubUnits + in_span, kIdescQK, uint32_t(s > 0));
                }
                rz::Tcgen05Commit<1>::execute(&pipe.s_full[qt][j % kSBufs]);
            };
            auto issue_pv = [&](int st, int j) {
                if (!leader) return;
                const uint32_t b0 = v_lo + uint32_t(st) * kKvTileUnits;
#pragma unroll
                for (int s = 0; s < Cfg::kPvSteps; ++s) {
                    const uint32_t b = b0 + uint32_t((s * Cfg::kMmaK * 128) >> 4);
                    const uint32_t acc = (s == 0) ? uint32_t(j != 0) : 1u;
                    if constexpr (kPSmem) {
                        const uint32_t off = uint32_t((s * 32) / 128) * kSubUnits + uint32_t(((s * 32) % 128) >> 4);
                        rz::Tcgen05MmaLo<!kFp8>::execute(tO, p_lo + uint32_t(j & 1) * kTileUnits + off, b, kIdescPV, acc);
                    } else {
                        rz::Tcgen05MmaLo<!kFp8>::execute_tmem_a(tO, tmem_base + uint32_t(qt * 128 + (j % kSBufs) * kN + s * 8), b, kIdescPV, acc);
                    }
                }
                rz::Tcgen05Commit<1>::execute(&pipe.o_done[qt][j & 1]);
            };
            long long dbg_w[4] = {0, 0, 0, 0};      // probes: cycles waiting for K / Q, V, P, other
            auto wait_or_report = [&](uint64_t* bar, uint32_t parity, uint32_t code, int kind = 3) {
                long long t0 = 0;
                if constexpr (kAttnProbes) t0 = clock64();
                const bool got = __all_sync(0xffffffffu, rz::BarrierWait::execute(bar, parity, abort_flag));
                if constexpr (kAttnProbes) dbg_w[kind] += clock64() - t0;
                if (got) return true;
                if (leader) attn_report(p, &pipe, rz::kRoleMma | code);
                return false;
            };
            const long long dbg_start = kAttnProbes ? clock64() : 0;
            int kst = 0, vst = 0;
            uint32_t kphase = 0, vphase = 0;
            auto next_k = [&]() { if (++kst == kStages) { kst = 0; kphase ^= 1u; } };
            auto next_v = [&]() { if (++vst == kStages) { vst = 0; vphase ^= 1u; } };
            // scores of KV tile jj (K at ring position kst), then this issuer's share of the slot release
            auto qk_step = [&](int jj) {
                if (!wait_or_report(&pipe.k_full[kst], kphase, rz::kBarFull, 0)) return false;
                if (jj == 0 && !wait_or_report(&pipe.q_full[qt], 0, rz::kBarFull, 0)) return false;
                if constexpr (kPSmem) {
                    if (jj > 0 && !wait_or_report(&pipe.s_free[qt], uint32_t((jj - 1) & 1), rz::kBarTmemEmpty)) return false;
                }
                rz::Tcgen05FenceAfter::execute();
                if (leader) attn_stamp(p, 12 + qt, jj);
                issue_qk(kst, jj);
                if (leader) rz::Tcgen05Commit<1>::execute(&pipe.k_empty[kst]);
                next_k();
                return true;
            };
            auto pv_step = [&](int j) {
                if (!wait_or_report(&pipe.v_full[vst], vphase, rz::kBarFull, 1)) return false;
                if (!wait_or_report(&pipe.p_full[qt][j & 1], uint32_t((j >> 1) & 1), rz::kBarOther, 2)) return false;
                rz::Tcgen05FenceAfter::execute();
                if (leader) attn_stamp(p, 10 + qt, j);
                issue_pv(vst, j);
                if (leader) rz::Tcgen05Commit<1>::execute(&pipe.v_empty[vst]);
                next_v();
                return true;
            };
            bool ok = true;
            if constexpr (kPSmem) {
                if (n > 0) ok = qk_step(0);
                for (int j = 0; j < n && ok; ++j) {
                    if (j + 1 < n) ok = qk_step(j + 1);
                    if (ok) ok = pv_step(j);
                }
            } else {
                for (int jj = 0; jj < kSBufs && jj < n && ok; ++jj) ok = qk_step(jj);
                for (int j = 0; j < n && ok; ++j) {
                    ok = pv_step(j);
                    if (ok && j + kSBufs < n) ok = qk_step(j + kSBufs);
                }
            }
#if defined(AXP_SM100_LATENCY_PROBES)
            if (leader && p.debug && blockIdx.x == unsigned(p.experiment >> 8)) {
                for (int i = 0; i < 4; ++i) p.debug[15 * 32 + 8 + qt * 5 + i] = (unsigned long long)dbg_w[i];
                p.debug[15 * 32 + 8 + qt * 5 + 4] = (unsigned long long)(clock64() - dbg_start);
            }
#endif
            // KV tiles only the other Q tile visits: K_j then V_j in tile order, as the producer refills them
            for (int j = n; j < n_max && ok; ++j) {
                if (!(ok = wait_or_report(&pipe.k_full[kst], kphase, rz::kBarFull))) break;
                if (leader) rz::BarrierArrive::execute(&pipe.k_empty[kst]);
                next_k();
                if (!(ok = wait_or_report(&pipe.v_full[vst], vphase, rz::kBarFull))) break;
                if (leader) rz::BarrierArrive::execute(&pipe.v_empty[vst]);
                next_v();
            }
        } else if (!p.two_issuers && warp == 9 && lane == 0) {
            // ------------------------------------------------------ MMA issuer ----
            // One lane runs the issue loop: a converged warp (32 lanes in every wait, lane 0 issuing) and one issuing
            // thread per Q tile both measured slower.
            const uint32_t tO[2] = {tmem_base + 256u, tmem_base + 384u};
            // S buffer b of Q tile qt: kN columns at qt * 128 + b * kN
            auto tS = [&](int qt, int b) { return tmem_base + uint32_t(qt * 128 + b * kN); };
            // Low descriptor words of the tiles; every MMA then costs the issuing thread two adds.
            const uint32_t q_lo = rz::sw128_desc_lo(rz::smem_u32(sQ), 16);
            const uint32_t k_lo = rz::sw128_desc_lo(rz::smem_u32(sK), 16);
            const uint32_t v_lo = rz::sw128_desc_lo(rz::smem_u32(sV), Cfg::kKvSubBytes);   // MN-major: next 128-byte span of d
            const uint32_t p_lo = rz::sw128_desc_lo(rz::smem_u32(sP), 16);
            constexpr uint32_t kTileUnits = Cfg::kTileBytes >> 4;               // descriptor address units are 16 bytes
            constexpr uint32_t kKvTileUnits = Cfg::kKvTileBytes >> 4;
            constexpr uint32_t kSubUnits = Cfg::kSubBytes >> 4;
            constexpr uint32_t kKvSubUnits = Cfg::kKvSubBytes >> 4;
            // S[qt][j % kSBufs] = Q[qt] . K[stage st]^T
            auto issue_qk = [&](int qt, int st, int j) {
                const uint32_t a0 = q_lo + uint32_t(qt) * kTileUnits;
                const uint32_t b0 = k_lo + uint32_t(st) * kKvTileUnits;
                const uint32_t d = tS(qt, j % kSBufs);
#pragma unroll
                for (int s = 0; s < Cfg::kSteps; ++s) {
                    // 32 bytes of the head dimension per step: inside a 128-byte span, then the next span
                    const uint32_t in_span = uint32_t(((s * 32) % 128) >> 4);
                    rz::Tcgen05MmaLo<!kFp8>::execute(d, a0 + uint32_t((s * 32) / 128) * kSubUnits + in_span,
                                                     b0 + uint32_t((s * 32) / 128) * kKvSubUnits + in_span, kIdescQK, uint32_t(s > 0));
                }
                rz::Tcgen05Commit<1>::execute(&pipe.s_full[qt][j % kSBufs]);
            };
            // O[qt] (+)= P . V[stage st]
            auto issue_pv = [&](int qt, int st, int j) {
                const uint32_t b0 = v_lo + uint32_t(st) * kKvTileUnits;
                const uint32_t d = tO[qt];
#pragma unroll
                for (int s = 0; s < Cfg::kPvSteps; ++s) {
                    // key rows [s*kMmaK, +kMmaK) of the V tile (128 bytes per row)
                    const uint32_t b = b0 + uint32_t((s * Cfg::kMmaK * 128) >> 4);
                    const uint32_t acc = (s == 0) ? uint32_t(j != 0) : 1u;
                    if constexpr (kPSmem) {
                        // P tile in shared memory, laid out like a Q tile: 32 bytes of keys per step
                        const uint32_t off = uint32_t((s * 32) / 128) * kSubUnits + uint32_t(((s * 32) % 128) >> 4);
                        rz::Tcgen05MmaLo<!kFp8>::execute(d, p_lo + uint32_t(qt * 2 + (j & 1)) * kTileUnits + off, b, kIdescPV, acc);
                    } else {
                        // P in tensor memory over the first columns of its S buffer; it advances 8 columns per step
                        rz::Tcgen05MmaLo<!kFp8>::execute_tmem_a(d, tS(qt, j % kSBufs) + uint32_t(s * 8), b, kIdescPV, acc);
                    }
                }
                rz::Tcgen05Commit<1>::execute(&pipe.o_done[qt][j & 1]);
            };
            auto wait_or_report = [&](uint64_t* bar, uint32_t parity, uint32_t code) {
                if (rz::BarrierWait::execute(bar, parity, abort_flag)) return true;
                attn_report(p, &pipe, rz::kRoleMma | code);
                return false;
            };
            auto tiles_of = [&](int qt) { return qt == 0 ? n0 : n1; };
            bool ok = n_max > 0;
            // K and V tiles are consumed at different steps: each has its own ring position
            int kst = 0, vst = 0;
            uint32_t kphase = 0, vphase = 0;
            auto next_k = [&]() { if (++kst == kStages) { kst = 0; kphase ^= 1u; } };
            auto next_v = [&]() { if (++vst == kStages) { vst = 0; vphase ^= 1u; } };
            // Q.K^T of KV tile jj for both Q tiles (K tile at ring position kst), then the slot goes back
            auto qk_step = [&](int jj, bool first) {
                if (!wait_or_report(&pipe.k_full[kst], kphase, rz::kBarFull)) return false;
                for (int qt = 0; qt < kQTiles; ++qt) {
                    if (jj < tiles_of(qt)) {
                        if (first && !wait_or_report(&pipe.q_full[qt], 0, rz::kBarFull)) return false;
                        if constexpr (kPSmem) {
                            // the softmax has taken the previous scores of this Q tile out of tensor memory
                            if (jj > 0 && !wait_or_report(&pipe.s_free[qt], uint32_t((jj - 1) & 1), rz::kBarTmemEmpty)) return false;
                        }
                        rz::Tcgen05FenceAfter::execute();
                        attn_stamp(p, 12 + qt, jj);
                        issue_qk(qt, kst, jj);
                    }
                }
                rz::Tcgen05Commit<1>::execute(&pipe.k_empty[kst]);
                next_k();
                return true;
            };
            auto pv_step = [&](int j) {
                if (!wait_or_report(&pipe.v_full[vst], vphase, rz::kBarFull)) return false;
                const int last_qt = (j < n1) ? 1 : 0;       // the last Q tile that reads this V tile
                bool k_ready = false;
                for (int qt = 0; qt < kQTiles; ++qt) {
                    if (j < tiles_of(qt)) {
                        if (!wait_or_report(&pipe.p_full[qt][j & 1], uint32_t((j >> 1) & 1), rz::kBarOther)) return false;
                        rz::Tcgen05FenceAfter::execute();
                        attn_stamp(p, 10 + qt, j);
                        issue_pv(qt, vst, j);
                        if (qt == last_qt) rz::Tcgen05Commit<1>::execute(&pipe.v_empty[vst]);
                        if constexpr (!kPSmem) {
                            // P lay over S buffer j % kSBufs: the next scores for that buffer follow the P.V in issue order
                            if (j + kSBufs < tiles_of(qt)) {
                                if (!k_ready && !wait_or_report(&pipe.k_full[kst], kphase, rz::kBarFull)) return false;
                                k_ready = true;
                                rz::Tcgen05FenceAfter::execute();
                                attn_stamp(p, 12 + qt, j + kSBufs);
                                issue_qk(qt, kst, j + kSBufs);
                            }
                        }
                    }
                }
                next_v();
                if constexpr (!kPSmem) {
                    if (k_ready) {
                        rz::Tcgen05Commit<1>::execute(&pipe.k_empty[kst]);
                        next_k();
                    }
                }
                return true;
            };
            if constexpr (kPSmem) {
                // S0' S1' as soon as the softmax has read S0 / S1 of the step, then PV0 PV1
                if (ok) ok = qk_step(0, true);
                for (int j = 0; j < n_max && ok; ++j) {
                    if (j + 1 < n_max) ok = qk_step(j + 1, false);
                    if (ok) ok = pv_step(j);
                }
            } else {
                // S of the first kSBufs steps, then per step PV0 S0' PV1 S1' (S' = scores of step j + kSBufs)
                for (int jj = 0; jj < kSBufs && jj < n_max && ok; ++jj) ok = qk_step(jj, jj == 0);
                for (int j = 0; j < n_max && ok; ++j) ok = pv_step(j);
            }
        }
    } else {
        // ------------------------------------ softmax / correction / epilogue ----
        rz::RegAlloc<kSoftmaxRegs>::execute();
        const int qt = warp >> 2;
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;
        const int q_tile_base = q_base + qt * kTileM;
        const int q = q_tile_base + row;
        const int qpos = stacked ? q % p.q_per_head : q;      // position of the query inside its head
        const int n = (qt == 0) ? n0 : n1;
        const uint32_t lane_addr = uint32_t(quarter * 32) << 16;
        const uint32_t tS0 = tmem_base + lane_addr + uint32_t(qt * 128);
        const uint32_t tO = tmem_base + lane_addr + uint32_t(256 + qt * 128);
        float c = p.scale * kLog2e;                       // scores -> log2 domain
        float out_scale = 1.0f;
        if constexpr (kFp8) {
            // stacked GQA heads: row r belongs to query head bh * group + r / q_per_head, which has its own Q descale
            const int qrow = q < p.Sq ? q : p.Sq - 1;
            const int q_head = stacked ? bh * (p.Sq / p.q_per_head) + qrow / p.q_per_head : bh;
            c *= __ldg(p.dq + q_head) * __ldg(p.dk + kvh);
            out_scale = __ldg(p.dv + kvh);
        }
        float m_used = -INFINITY;
        float l = 0.0f;
        bool ok = true;
        long long dbg_wait = 0, dbg_t0 = 0, dbg_first = 0;
        long long dbg_ph[4] = {0, 0, 0, 0};      // probes: cycles in S read, maximum / rescale, exponentials (+ turn wait), hand-over
        for (int j = 0; j < n; ++j) {
            const uint32_t tS = tS0 + uint32_t((j % kSBufs) * kN);     // this step's S buffer (P goes over its first columns)
            if constexpr (kAttnProbes) dbg_t0 = clock64();
            ok = __all_sync(0xffffffffu, rz::BarrierWait::execute(&pipe.s_full[qt][j % kSBufs], uint32_t((j / kSBufs) & 1), abort_flag));
            if constexpr (kAttnProbes) {
                if (j == 0) dbg_first = clock64();
                else dbg_wait += clock64() - dbg_t0;
                dbg_t0 = clock64();
            }
            if (!ok) {
                if (lane == 0) attn_report(p, &pipe, rz::kRoleSoftmax | rz::kBarTmemFull);
                break;
            }
            rz::Tcgen05FenceAfter::execute();
            if (lane == 0 && quarter == 0) attn_stamp(p, qt * 5 + 0, j);     // S seen
            const int k0 = (j_lo + j) * kN;
            // the first row of the tile (stacked heads: a first query of some head) sees the fewest keys
            const bool need_mask = (p.causal && !rz::causal_valid((stacked ? 0 : q_tile_base) + causal_off, k0 + kN - 1)) || (k0 + kN > p.Skv);
            auto mask32 = [&](uint32_t (&v)[32], int col0) {
                if (need_mask) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const int kpos = k0 + col0 + i;
                        if ((p.causal && !rz::causal_valid(qpos + causal_off, kpos)) || kpos >= p.Skv) v[i] = 0xff800000u;   // -inf
                    }
                }
            };
            // ---- the kN scores of this row go to registers once; row maximum with three-input max ----
            float mx;
            uint32_t v0[32], v1[32], v2[32], v3[32];
            {
                rz::TmemLoad32x32::execute(tS, v0);
                rz::TmemLoad32x32::execute(tS + 32u, v1);
                if constexpr (kN == 128) {
                    rz::TmemLoad32x32::execute(tS + 64u, v2);
                    rz::TmemLoad32x32::execute(tS + 96u, v3);
                }
                rz::TmemLoadWait::execute(v0);
                rz::TmemLoadWait::execute(v1);
                if constexpr (kN == 128) {
                    rz::TmemLoadWait::execute(v2);
                    rz::TmemLoadWait::execute(v3);
                }
                if constexpr (kAttnProbes) { const long long t = clock64(); dbg_ph[0] += t - dbg_t0; dbg_t0 = t; }
                if constexpr (kPSmem) {
                    // S is in registers: its tensor-memory columns may take the next Q.K^T of this Q tile
                    rz::Tcgen05FenceBefore::execute();
                    __syncwarp();
                    if (lane == 0) rz::BarrierArrive::execute(&pipe.s_free[qt]);
                    if (lane == 0 && quarter == 0) attn_stamp(p, qt * 5 + 2, j);     // S in registers, columns released
                }
                mask32(v0, 0);
                mask32(v1, 32);
                float m0 = __uint_as_float(v0[0]), m1 = __uint_as_float(v1[0]);
#pragma unroll
                for (int i = 1; i < 32; i += 2) {
                    const int i2 = (i + 1 < 32) ? i + 1 : i;
                    m0 = rz::max3_f32(m0, __uint_as_float(v0[i]), __uint_as_float(v0[i2]));
                    m1 = rz::max3_f32(m1, __uint_as_float(v1[i]), __uint_as_float(v1[i2]));
                }
                mx = fmaxf(m0, m1);
                if constexpr (kN == 128) {
                    mask32(v2, 64);
                    mask32(v3, 96);
                    float m2 = __uint_as_float(v2[0]), m3 = __uint_as_float(v3[0]);
#pragma unroll
                    for (int i = 1; i < 32; i += 2) {
                        const int i2 = (i + 1 < 32) ? i + 1 : i;
                        m2 = rz::max3_f32(m2, __uint_as_float(v2[i]), __uint_as_float(v2[i2]));
                        m3 = rz::max3_f32(m3, __uint_as_float(v3[i]), __uint_as_float(v3[i2]));
                    }
                    mx = fmaxf(mx, fmaxf(m2, m3));
                }
            }
            if (j == 0) {
                m_used = (mx == -INFINITY) ? 0.0f : mx;
            } else {
                const bool grow = (mx - m_used) * c > p.rescale_thr;
                if (__any_sync(0xffffffffu, grow)) {
                    float factor = 1.0f;
                    if (grow) {
                        factor = rz::exp2_approx((m_used - mx) * c);
                        m_used = mx;
                        l *= factor;
                    }
                    // O of this Q tile must be final for step j-1 before it is rescaled in place
                    ok = __all_sync(0xffffffffu,
                                    rz::BarrierWait::execute(&pipe.o_done[qt][(j - 1) & 1], uint32_t(((j - 1) >> 1) & 1), abort_flag));
                    if (!ok) {
                        if (lane == 0) attn_report(p, &pipe, rz::kRoleCorrection | rz::kBarOther);
                        break;
                    }
                    rz::Tcgen05FenceAfter::execute();
#pragma unroll 1
                    for (int cc = 0; cc < 4; ++cc) {
                        uint32_t v[32];
                        rz::TmemLoad32x32::execute(tO + uint32_t(cc * 32), v);
                        rz::TmemLoadWait::execute(v);
#pragma unroll
                        for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * factor);
                        rz::TmemStore32x32::execute(tO + uint32_t(cc * 32), v);
                    }
                }
            }
            if constexpr (kAttnProbes) { const long long t = clock64(); dbg_ph[1] += t - dbg_t0; dbg_t0 = t; }
            if (lane == 0 && quarter == 0) attn_stamp(p, qt * 5 + 1, j);     // maximum known
            // ---- P = exp2(s*c - m*c): packed fp32 pairs for scale/shift and row sums; of every eight pairs the ones in
            //      kPolyMask take the polynomial on the FMA pipe, the others the SFU.  P leaves in 16-column blocks:
            //      shared memory (kPSmem) or tensor memory over the first columns of S ----
            const float neg = -m_used * c;
            const unsigned long long c2 = rz::pack_f32x2(c, c), neg2 = rz::pack_f32x2(neg, neg);
            unsigned long long sum_a = rz::pack_f32x2(0.0f, 0.0f), sum_b = sum_a;
            if constexpr (kPSmem) {
                static_assert(!kPSmem || kFp8, "P through shared memory is realised for E4M3 only");
                // buffer j & 1 of this Q tile was last read by the P.V of step j - 2
                if (j >= 2) {
                    ok = __all_sync(0xffffffffu, rz::BarrierWait::execute(&pipe.o_done[qt][j & 1], uint32_t(((j >> 1) - 1) & 1), abort_flag));
                    if (!ok) {
                        if (lane == 0) attn_report(p, &pipe, rz::kRoleSoftmax | rz::kBarOther);
                        break;
                    }
                }
            }
            // kPSmem: row `row` of the K-major 128-byte-swizzled tile, 16-byte chunk b sits at chunk b ^ (row & 7)
            uint8_t* prow = sP + (qt * 2 + (j & 1)) * Cfg::kTileBytes + row * 128;
            const int sw = row & 7;
            uint32_t pk[32];
            auto block16 = [&](uint32_t (&v)[32], int o16, int b) {
                float e[16];
                rz::RowSoftmaxExp2::execute<kPolyMask>(v, o16, c2, neg2, sum_a, sum_b, e);
                if constexpr (kFp8 && kPSmem) {
                    uint32_t w[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) w[i] = rz::PackE4m3x4::execute(e[4 * i], e[4 * i + 1], e[4 * i + 2], e[4 * i + 3]);
                    *reinterpret_cast<uint4*>(prow + ((b ^ sw) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
                } else if constexpr (kFp8) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) pk[(b & 3) * 4 + i] = rz::PackE4m3x4::execute(e[4 * i], e[4 * i + 1], e[4 * i + 2], e[4 * i + 3]);
                    if ((b & 3) == 3) {
                        uint32_t(&half)[16] = *reinterpret_cast<uint32_t(*)[16]>(&pk[0]);
                        rz::TmemStore32x16::execute(tS + uint32_t((b >> 2) * 16), half);
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 8; ++i) pk[(b & 3) * 8 + i] = rz::PackBf16x2::execute(e[2 * i], e[2 * i + 1]);
                    if ((b & 3) == 3) rz::TmemStore32x32::execute(tS + uint32_t((b >> 2) * 32), pk);
                }
            };
            block16(v0, 0, 0);
            block16(v0, 16, 1);
            block16(v1, 0, 2);
            block16(v1, 16, 3);
            if (lane == 0 && quarter == 0) attn_stamp(p, qt * 5 + 3, j);     // first 64 columns of P issued
            if constexpr (kN == 128) {
                block16(v2, 0, 4);
                block16(v2, 16, 5);
                block16(v3, 0, 6);
                block16(v3, 16, 7);
            }
            if constexpr (kAttnProbes) { const long long t = clock64(); dbg_ph[2] += t - dbg_t0; dbg_t0 = t; }
            {
                float a0, a1, b0, b1;
                rz::unpack_f32x2(sum_a, a0, a1);
                rz::unpack_f32x2(sum_b, b0, b1);
                l += (a0 + a1) + (b0 + b1);
            }
            if constexpr (kPSmem) {
                rz::AsyncProxyFence::execute();
            } else {
                rz::TmemStoreWait::execute();
                rz::Tcgen05FenceBefore::execute();
            }
            __syncwarp();
            if (lane == 0) rz::BarrierArrive::execute(&pipe.p_full[qt][j & 1]);
            if constexpr (kAttnProbes) { const long long t = clock64(); dbg_ph[3] += t - dbg_t0; dbg_t0 = t; }
            if (lane == 0 && quarter == 0) attn_stamp(p, qt * 5 + 4, j);     // P handed to the issuer
        }
#if defined(AXP_SM100_LATENCY_PROBES)
        if (lane == 0 && quarter == 0 && p.debug && blockIdx.x == unsigned(p.experiment >> 8)) {
            p.debug[15 * 32 + qt * 2 + 0] = (unsigned long long)dbg_wait;                 // cycles waiting for S, steps 1..n-1
            p.debug[15 * 32 + qt * 2 + 1] = (unsigned long long)(clock64() - dbg_first);  // cycles from first S to loop end
            for (int i = 0; i < 4; ++i) p.debug[15 * 32 + 20 + qt * 4 + i] = (unsigned long long)dbg_ph[i];
        }
#endif
        if (lane == 0 && quarter == 0) attn_stamp(p, 14, 2 + qt * 3);       // softmax loop left
        if (ok && n > 0) {
            ok = __all_sync(0xffffffffu, rz::BarrierWait::execute(&pipe.o_done[qt][(n - 1) & 1], uint32_t(((n - 1) >> 1) & 1), abort_flag));
            if (lane == 0 && quarter == 0) attn_stamp(p, 14, 3 + qt * 3);   // last P.V complete
            if (!ok) {
                if (lane == 0) attn_report(p, &pipe, rz::kRoleEpilogue | rz::kBarOther);
            } else {
                rz::Tcgen05FenceAfter::execute();
                const float inv = out_scale / l;
                const bool row_ok = q < p.Sq;
                __nv_bfloat16* orow = static_cast<__nv_bfloat16*>(p.O) + ((long long)bh * p.Sq + q) * kHeadDim;
                // The finished O tile leaves through shared memory and one TMA store per 64 columns (a row-per-thread
                // store to global memory took 2.4 us per CTA): it is staged, swizzled like a Q tile, where this Q tile's
                // Q (bf16) or P buffers (E4M3, P through shared memory) lay - every MMA that read them has completed.
                constexpr bool kStageO = !kFp8 || kPSmem;
                uint8_t* so = kFp8 ? sP + qt * 2 * Cfg::kTileBytes : sQ + qt * Cfg::kTileBytes;
                const bool staged = kStageO && !p.partial;
                // split-KV: the partial result of this KV share, row `prow` of [splits][heads][Sq]
                const long long prow = ((long long)blockIdx.z * p.num_heads + (bh - p.bh_begin)) * p.Sq + q;
#pragma unroll 1
                for (int cc = 0; cc < 4; ++cc) {
                    uint32_t v[32];
                    rz::TmemLoad32x32::execute(tO + uint32_t(cc * 32), v);
                    rz::TmemLoadWait::execute();
                    if (row_ok && p.partial) {
                        float4* dst = reinterpret_cast<float4*>(p.part_o + prow * kHeadDim + cc * 32);
#pragma unroll
                        for (int g = 0; g < 8; ++g)
                            dst[g] = make_float4(__uint_as_float(v[g * 4 + 0]) * out_scale, __uint_as_float(v[g * 4 + 1]) * out_scale,
                                                 __uint_as_float(v[g * 4 + 2]) * out_scale, __uint_as_float(v[g * 4 + 3]) * out_scale);
                    } else if (row_ok || staged) {
#pragma unroll
                        for (int g = 0; g < 4; ++g) {
                            uint4 o;
                            o.x = rz::PackBf16x2::execute(__uint_as_float(v[g * 8 + 0]) * inv, __uint_as_float(v[g * 8 + 1]) * inv);
                            o.y = rz::PackBf16x2::execute(__uint_as_float(v[g * 8 + 2]) * inv, __uint_as_float(v[g * 8 + 3]) * inv);
                            o.z = rz::PackBf16x2::execute(__uint_as_float(v[g * 8 + 4]) * inv, __uint_as_float(v[g * 8 + 5]) * inv);
                            o.w = rz::PackBf16x2::execute(__uint_as_float(v[g * 8 + 6]) * inv, __uint_as_float(v[g * 8 + 7]) * inv);
                            if (staged) {
                                // columns [cc*32 + g*8, +8): 128-byte span (cc*32 + g*8) / 64, 16-byte chunk ((cc*32 + g*8) % 64) / 8
                                const int span = (cc * 32 + g * 8) / 64, chunk = ((cc * 32 + g * 8) % 64) / 8;
                                *reinterpret_cast<uint4*>(so + span * Cfg::kSubBytes + row * 128 + ((chunk ^ (row & 7)) << 4)) = o;
                            } else {
                                *reinterpret_cast<uint4*>(orow + cc * 32 + g * 8) = o;
                            }
                        }
                    }
                }
                if (staged) {
                    rz::AsyncProxyFence::execute();
                    rz::NamedBarrierSync::execute(1u + uint32_t(qt), kTileM);       // the four warps of this Q tile
                    if (quarter == 0 && lane == 0) {
                        rz::BulkTmaStore3D::execute(&tmO, so, 0, q_tile_base, bh);
                        rz::BulkTmaStore3D::execute(&tmO, so + Cfg::kSubBytes, 64, q_tile_base, bh);
                        rz::BulkStoreCommit::execute();
                        rz::BulkStoreWaitRead<0>::execute();       // shared memory stays until the store has read it
                    }
                }
                if (lane == 0 && quarter == 0) attn_stamp(p, 14, 4 + qt * 3);   // O stored
                if (row_ok && p.partial) p.part_ml[prow] = make_float2(m_used * c, l);
                else if (row_ok && p.LSE) p.LSE[(long long)bh * p.Sq + q] = (m_used * c + log2f(l)) * kLn2;
            }
        } else if (ok && p.partial && q < p.Sq) {
            // no key of this KV share is visible to the row: an empty partial result
            p.part_ml[((long long)blockIdx.z * p.num_heads + (bh - p.bh_begin)) * p.Sq + q] = make_float2(-INFINITY, 0.0f);
        }
    }

    rz::Tcgen05FenceBefore::execute();
    __syncthreads();
    if (threadIdx.x == 0) attn_stamp(p, 14, 8);       // all roles done
    if (warp == 9) {
        rz::Tcgen05FenceAfter::execute();
        rz::TmemDealloc<1>::execute(tmem_base, 512);
        if (lane == 0) attn_stamp(p, 14, 9);          // tensor memory returned
    }
}

// Split-KV combine: row r of the output from the partial results of the KV shares,
//   m = max_z m_z,  w_z = exp2(m_z - m),  O = sum_z w_z O_z / sum_z w_z l_z,  LSE = (m + log2(sum_z w_z l_z)) ln 2.
// One warp per row, four head-dimension columns per lane; shares with no visible key (l = 0) are skipped.
// Share z has its accumulators at part_o + z * o_stride (floats) and its (m, l) at part_ml + z * ml_stride (float2).
__global__ void __launch_bounds__(256) attn_splitkv_combine_kernel(const float* __restrict__ part_o, const float2* __restrict__ part_ml,
                                                                   long long o_stride, long long ml_stride,
                                                                   __nv_bfloat16* __restrict__ O, float* __restrict__ LSE, long long rows,
                                                                   int splits, long long o_row0) {
    const long long r = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (r >= rows) return;
    float m = -INFINITY;
    for (int z = 0; z < splits; ++z) {
        const float2 ml = part_ml[(long long)z * ml_stride + r];
        if (ml.y > 0.0f) m = fmaxf(m, ml.x);
    }
    float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    float den = 0.0f;
    for (int z = 0; z < splits; ++z) {
        const float2 ml = part_ml[(long long)z * ml_stride + r];
        if (ml.y > 0.0f) {
            const float w = exp2f(ml.x - m);
            const float4 o = reinterpret_cast<const float4*>(part_o + (long long)z * o_stride + r * kHeadDim)[lane];
            acc.x = fmaf(w, o.x, acc.x);
            acc.y = fmaf(w, o.y, acc.y);
            acc.z = fmaf(w, o.z, acc.z);
            acc.w = fmaf(w, o.w, acc.w);
            den = fmaf(w, ml.y, den);
        }
    }
    const float inv = den > 0.0f ? 1.0f / den : 0.0f;
    uint2 out;
    out.x = rz::PackBf16x2::execute(acc.x * inv, acc.y * inv);
    out.y = rz::PackBf16x2::execute(acc.z * inv, acc.w * inv);
    reinterpret_cast<uint2*>(O + (o_row0 + r) * kHeadDim)[lane] = out;
    if (LSE && lane == 0) LSE[o_row0 + r] = den > 0.0f ? (m + log2f(den)) * kLn2 : -INFINITY;
}

// ------------------------------------------------------------------------------------------------------------------
// Decode attention (bf16 or E4M3, up to 16 query rows per KV head and call): the operands are swapped.
// S^T = K . Q^T puts the 128 keys of a KV tile on the 128 tensor-memory lanes and the (at most 16) query rows on 16
// columns, so every softmax thread owns one key and 16 scores instead of one mostly empty query row and 128 scores;
// O^T = V^T . P^T accumulates [128 head-dim lanes x 16 query columns].  P^T goes through shared memory (K-major B
// operand), V is used where it lies as an MN-major A operand.  One CTA per (KV head, KV share); the result leaves
// as the partial results the split-KV combine kernel reads or, with one KV share, normalised as O and LSE.
constexpr int kDecQ = 16;             // query rows per CTA (N of both MMAs)
constexpr int kDecKeys = 128;         // keys per KV tile (M of S^T, K of O^T)
constexpr int kDecThreads = 192;      // warps 0-3 softmax (one key per thread), warp 4 TMA producer, warp 5 MMA issuer
constexpr int kDecMaxStages = 3;      // barrier array size in DecodePipe
template <bool kFp8>
struct DecCfg {
    static constexpr int kSpans = kFp8 ? 1 : 2;                    // 128-byte spans per row of D (and per P^T row of 128 keys)
    static constexpr int kSpanElems = kFp8 ? 128 : 64;
    // K and V ring slots.  bf16: one CTA per SM with 96 KiB of K and of V in flight.  E4M3 tiles are half as large
    // and their per-tile chain (scores, maxima exchange, exponentials, P^T, MMAs) takes as long as for bf16, so two
    // CTAs share an SM (48 KiB of K and of V each) and fill each other's waits.
    static constexpr int kStages = 3;
    static constexpr int kCtasPerSm = kFp8 ? 2 : 1;
    static constexpr int kQpRegion = kFp8 ? 8192 : 16384;          // Q and the two P^T buffers
    static constexpr int kQBytes = kSpans * kDecQ * 128;           // Q: spans of [16 rows x 128 B]
    static constexpr int kPBytes = kSpans * kDecQ * 128;           // P^T: spans of [16 rows x 128 B]
    static constexpr int kKvSpanBytes = kDecKeys * 128;            // [128 keys x 128 B]
    static constexpr int kKvBytes = kSpans * kKvSpanBytes;         // K or V tile
    static constexpr int kMmaSteps = kFp8 ? 4 : 8;                 // MMAs per product: 32 bytes of the contraction each
    static constexpr int kSmem = 1024 + kQpRegion + 2 * kStages * kKvBytes;     // alignment slack, Q and P^T, K and V rings
    static_assert(kQBytes + 2 * kPBytes <= kQpRegion && kCtasPerSm * (kSmem + 2048) <= 227 * 1024, "shared memory budget");
};

struct DecodeParams {
    float* part_o;         // [shares][heads][rows][128]
    float2* part_ml;       // [shares][heads][rows]
    int rows;              // query rows per (stacked) head, <= 16
    int q_per_head;        // row r is query r % q_per_head of group member r / q_per_head
    int Skv;
    int Hq, Hkv;           // after stacking
    int causal;
    int causal_off;        // query position i sees keys <= i + causal_off
    int bh_begin;
    int num_heads;
    int tiles_per_split;
    float scale;
    uint32_t* status;
    const float* dq;       // E4M3: descales per query head [B*Hq before stacking], per KV head
    const float* dk;
    const float* dv;
    __nv_bfloat16* O;      // direct mode (one KV share, no partial results): [heads of the call][rows][128], normalised
    float* LSE;            // direct mode: [heads of the call][rows] or null
    int direct;
};

struct DecodePipe {
    uint64_t q_full;
    uint64_t k_full[kDecMaxStages], k_empty[kDecMaxStages], v_full[kDecMaxStages], v_empty[kDecMaxStages];
    uint64_t s_full[2];    // S^T of step j: s_full[j & 1], phase j >> 1
    uint64_t p_full[2];    // P^T of step j written by the four softmax warps
    uint64_t pv_done[2];   // O^T += V^T . P^T of step j complete (P buffer j & 1 free, O final for step j)
    uint64_t mx_bar[2];    // the four warps' tile maxima of step j are in mx[j & 1]
    uint64_t l_bar;        // the four warps' row sums are in lsum
    uint32_t tmem_base;
    uint32_t abort_flag;
    alignas(16) float mx[2][4][kDecQ];      // read as float4
    alignas(16) float lsum[4][kDecQ];
};

template <bool kFp8>
__global__ void __launch_bounds__(kDecThreads, DecCfg<kFp8>::kCtasPerSm)
attn_decode_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, const DecodeParams p) {
    using Cfg = DecCfg<kFp8>;
    constexpr int kDecStages = Cfg::kStages, kDecQBytes = Cfg::kQBytes, kDecPBytes = Cfg::kPBytes, kDecKvBytes = Cfg::kKvBytes;
    constexpr uint32_t kFmt = kFp8 ? 0u : 1u;
    constexpr uint32_t kIdescQK = rz::make_instr_desc(kFmt, kFmt, false, false, kDecKeys, kDecQ);   // S^T: A = K (K-major), B = Q (K-major)
    constexpr uint32_t kIdescPV = rz::make_instr_desc(kFmt, kFmt, true, false, kHeadDim, kDecQ);    // O^T: A = V (MN-major), B = P^T (K-major)
    extern __shared__ uint8_t dyn_smem_raw[];
    __shared__ DecodePipe pipe;
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(dyn_smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sQ = smem;                                    // 4 KiB (E4M3: 2 KiB)
    uint8_t* sP = sQ + kDecQBytes;                         // two P^T buffers of the same size
    uint8_t* sK = smem + Cfg::kQpRegion;                   // ring slots start 1024-byte aligned
    uint8_t* sV = sK + kDecStages * kDecKvBytes;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    volatile uint32_t* abort_flag = &pipe.abort_flag;
    auto report = [&](uint32_t code) {
        *reinterpret_cast<volatile uint32_t*>(&pipe.abort_flag) = 1u;
        if (p.status) atomicOr(p.status, rz::kStatusError | code);
    };

    const int head_idx = int(blockIdx.x);
    const int bh = p.bh_begin + head_idx;
    const int batch = bh / p.Hq;
    const int kvh = batch * p.Hkv + (bh - batch * p.Hq) / (p.Hq / p.Hkv);
    // KV tiles of this CTA's share: the last key any row sees bounds the tiles under the causal mask
    const int j_lo = int(blockIdx.z) * p.tiles_per_split;
    int n_all = (p.Skv + kDecKeys - 1) / kDecKeys;
    if (p.causal) {
        const long long last_k = (long long)(p.q_per_head - 1) + p.causal_off;
        const long long vis = last_k < 0 ? 0 : last_k / kDecKeys + 1;
        if (vis < n_all) n_all = int(vis);
    }
    int n = n_all - j_lo;
    n = n < 0 ? 0 : (n < p.tiles_per_split ? n : p.tiles_per_split);

    auto load_kv = [&](const CUtensorMap* tm, uint8_t* dst, int j, uint64_t* bar) {
        rz::BarrierExpectTx::execute(bar, kDecKvBytes);
        for (int sp = 0; sp < Cfg::kSpans; ++sp)
            rz::BulkTmaCopy3D::execute(tm, dst + sp * Cfg::kKvSpanBytes, sp * Cfg::kSpanElems, (j_lo + j) * kDecKeys, kvh, bar);
    };
    const int n_first = n < kDecStages ? n : kDecStages;
    if (warp == 4 && lane == 0) {
        rz::PrefetchTensorMap::execute(&tmQ);
        rz::PrefetchTensorMap::execute(&tmK);
        rz::PrefetchTensorMap::execute(&tmV);
        rz::BarrierInit::execute(&pipe.q_full, 1);
        for (int s = 0; s < kDecStages; ++s) {
            rz::BarrierInit::execute(&pipe.k_full[s], 1);
            rz::BarrierInit::execute(&pipe.k_empty[s], 1);
            rz::BarrierInit::execute(&pipe.v_full[s], 1);
            rz::BarrierInit::execute(&pipe.v_empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            rz::BarrierInit::execute(&pipe.s_full[b], 1);
            rz::BarrierInit::execute(&pipe.p_full[b], 4);
            rz::BarrierInit::execute(&pipe.pv_done[b], 1);
            rz::BarrierInit::execute(&pipe.mx_bar[b], 4);
        }
        rz::BarrierInit::execute(&pipe.l_bar, 4);
        pipe.abort_flag = 0;
        rz::BarrierInitFence::execute();
        if (n > 0) {
            rz::BarrierExpectTx::execute(&pipe.q_full, kDecQBytes);
            for (int sp = 0; sp < Cfg::kSpans; ++sp)
                rz::BulkTmaCopy3D::execute(&tmQ, sQ + sp * kDecQ * 128, sp * Cfg::kSpanElems, 0, bh, &pipe.q_full);
        }
        for (int j = 0; j < n_first; ++j) {
            load_kv(&tmK, sK + j * kDecKvBytes, j, &pipe.k_full[j]);
            load_kv(&tmV, sV + j * kDecKvBytes, j, &pipe.v_full[j]);
        }
    }
    if (warp == 5) rz::TmemAlloc<1>::execute(&pipe.tmem_base, 64);
    rz::Tcgen05FenceBefore::execute();
    __syncthreads();
    rz::Tcgen05FenceAfter::execute();
    const uint32_t tmem_base = pipe.tmem_base;
    const uint32_t tO = tmem_base + 32u;          // S^T buffers at columns 0 and 16, O^T at 32

    if (warp == 4) {
        if (lane == 0) {
            // ---------------------------------------------------- TMA producer ----
            int st = n_first == kDecStages ? 0 : n_first;
            uint32_t phase = n_first == kDecStages ? 1u : 0u;
            bool ok = true;
            for (int j = n_first; j < n && ok; ++j) {
                if (!rz::BarrierWait::execute(&pipe.k_empty[st], phase ^ 1u, abort_flag)) { report(rz::kRoleProducer | rz::kBarEmpty); ok = false; break; }
                load_kv(&tmK, sK + st * kDecKvBytes, j, &pipe.k_full[st]);
                if (!rz::BarrierWait::execute(&pipe.v_empty[st], phase ^ 1u, abort_flag)) { report(rz::kRoleProducer | rz::kBarEmpty); ok = false; break; }
                load_kv(&tmV, sV + st * kDecKvBytes, j, &pipe.v_full[st]);
                if (++st == kDecStages) { st = 0; phase ^= 1u; }
            }
            // every requested tile has been consumed (its MMAs complete) before shared memory goes away
            for (int s = 0; s < kDecStages && ok; ++s) {
                if (!rz::BarrierWait::execute(&pipe.k_empty[st], phase ^ 1u, abort_flag) ||
                    !rz::BarrierWait::execute(&pipe.v_empty[st], phase ^ 1u, abort_flag)) { report(rz::kRoleProducer | rz::kBarEmpty); ok = false; }
                if (++st == kDecStages) { st = 0; phase ^= 1u; }
            }
        }
    } else if (warp == 5) {
        if (n > 0) {
            // ------------------------------------------------------ MMA issuer ----
            // the whole warp runs the loop (waits are votes of all lanes), one elected lane issues
            const bool elected = rz::elect_one();
            const uint32_t q_lo = rz::sw128_desc_lo(rz::smem_u32(sQ), 16);
            const uint32_t k_lo = rz::sw128_desc_lo(rz::smem_u32(sK), 16);
            const uint32_t v_lo = rz::sw128_desc_lo(rz::smem_u32(sV), kDecKeys * 128);      // MN-major: next 64 head-dim columns 16 KiB further
            const uint32_t p_lo = rz::sw128_desc_lo(rz::smem_u32(sP), 16);
            constexpr uint32_t kKvUnits = kDecKvBytes >> 4, kKvSpanUnits = (kDecKeys * 128) >> 4, kQSpanUnits = (kDecQ * 128) >> 4;
            auto wait_or_report = [&](uint64_t* bar, uint32_t parity, uint32_t code) {
                if (__all_sync(0xffffffffu, rz::BarrierWait::execute(bar, parity, abort_flag))) return true;
                if (elected) report(rz::kRoleMma | code);
                return false;
            };
            int kst = 0, vst = 0;
            uint32_t kphase = 0, vphase = 0;
            auto qk = [&](int j) {
                if (!wait_or_report(&pipe.k_full[kst], kphase, rz::kBarFull)) return false;
                rz::Tcgen05FenceAfter::execute();
                const uint32_t a0 = k_lo + uint32_t(kst) * kKvUnits;
#pragma unroll
                for (int s = 0; s < Cfg::kMmaSteps && elected; ++s)      // 32 bytes of the head dimension per MMA
                    rz::Tcgen05MmaLo<!kFp8>::execute(tmem_base + uint32_t((j & 1) * kDecQ), a0 + uint32_t(s / 4) * kKvSpanUnits + uint32_t(s & 3) * 2u,
                                                    q_lo + uint32_t(s / 4) * kQSpanUnits + uint32_t(s & 3) * 2u, kIdescQK, uint32_t(s > 0));
                if (elected) {
                    rz::Tcgen05Commit<1>::execute(&pipe.s_full[j & 1]);
                    rz::Tcgen05Commit<1>::execute(&pipe.k_empty[kst]);
                }
                if (++kst == kDecStages) { kst = 0; kphase ^= 1u; }
                return true;
            };
            auto pv = [&](int j) {
                if (!wait_or_report(&pipe.v_full[vst], vphase, rz::kBarFull)) return false;
                if (!wait_or_report(&pipe.p_full[j & 1], uint32_t((j >> 1) & 1), rz::kBarOther)) return false;
                rz::Tcgen05FenceAfter::execute();
                const uint32_t a0 = v_lo + uint32_t(vst) * kKvUnits;
                const uint32_t b0 = p_lo + uint32_t(j & 1) * (kDecPBytes >> 4);
#pragma unroll
                for (int s = 0; s < Cfg::kMmaSteps && elected; ++s)      // 16 (E4M3: 32) keys per MMA: as many 128-byte rows further in V, 32 B further in a P^T row
                    rz::Tcgen05MmaLo<!kFp8>::execute(tO, a0 + uint32_t(s) * (kFp8 ? 256u : 128u), b0 + uint32_t(s / 4) * kQSpanUnits + uint32_t(s & 3) * 2u, kIdescPV,
                                                    uint32_t(j > 0 || s > 0));
                if (elected) {
                    rz::Tcgen05Commit<1>::execute(&pipe.pv_done[j & 1]);
                    rz::Tcgen05Commit<1>::execute(&pipe.v_empty[vst]);
                }
                if (++vst == kDecStages) { vst = 0; vphase ^= 1u; }
                return true;
            };
            bool ok = wait_or_report(&pipe.q_full, 0, rz::kBarFull);
            if (ok) ok = qk(0);
            for (int j = 0; j < n && ok; ++j) {
                // S^T buffer (j + 1) & 1 was read by the softmax of step j - 1 before its P^T arrived, which P.V of step j - 1 waited for
                if (j + 1 < n) ok = qk(j + 1);
                if (ok) ok = pv(j);
            }
        }
    } else {
        // ------------------------------------------- softmax: one key per thread ----
        const int t = threadIdx.x;                       // key inside the tile = tensor-memory lane
        const uint32_t lane_addr = uint32_t(warp * 32) << 16;
        const float c0 = p.scale * kLog2e;
        // scores -> log2 domain; E4M3: times the Q descale of the row's own query head and the K descale
        float cq[kFp8 ? kDecQ : 1];
        float out_scale = 1.0f;
        if constexpr (kFp8) {
            const float dk = __ldg(p.dk + kvh);
            const int members = p.rows / p.q_per_head;           // stacked query heads of this KV head
#pragma unroll
            for (int q = 0; q < kDecQ; ++q) {
                const int member = q < p.rows ? q / p.q_per_head : 0;
                cq[q] = c0 * __ldg(p.dq + bh * members + member) * dk;
            }
            out_scale = __ldg(p.dv + kvh);
        } else {
            cq[0] = c0;
        }
        auto c_of = [&](int q) { return kFp8 ? cq[q] : cq[0]; };
        float ref[kDecQ];                                 // per query row: the reference (a running maximum) the exponentials are taken against
        float l[kDecQ];                                   // this thread's share of the row sums
#pragma unroll
        for (int q = 0; q < kDecQ; ++q) { ref[q] = 0.0f; l[q] = 0.0f; }
        bool ok = true;
        auto wait_or_report = [&](uint64_t* bar, uint32_t parity, uint32_t code) {
            const bool got = __all_sync(0xffffffffu, rz::BarrierWait::execute(bar, parity, abort_flag));
            if (!got && lane == 0) report(rz::kRoleSoftmax | code);
            return got;
        };
        for (int j = 0; j < n && ok; ++j) {
            if (!(ok = wait_or_report(&pipe.s_full[j & 1], uint32_t((j >> 1) & 1), rz::kBarTmemFull))) break;
            rz::Tcgen05FenceAfter::execute();
            uint32_t v[kDecQ];
            rz::TmemLoad32x16::execute(tmem_base + lane_addr + uint32_t((j & 1) * kDecQ), v);
            rz::TmemLoadWait::execute(v);
            // masks: keys past the end of the sequence (their K rows were zero-filled) and, under the causal mask,
            // keys after the query's position
            const int key = (j_lo + j) * kDecKeys + t;
            const bool tail = key >= p.Skv;
            const bool diag = p.causal && (j_lo + j + 1) * kDecKeys - 1 > p.causal_off;      // some row may not see the tile's last key
            if (tail || diag) {
#pragma unroll
                for (int q = 0; q < kDecQ; ++q) {
                    const int qpos = q % p.q_per_head;
                    if (tail || (p.causal && key > qpos + p.causal_off)) v[q] = 0xff800000u;   // -inf
                }
            }
            // tile maxima per query row over the 128 keys: warp reduction on an order-preserving integer image, then
            // the four warps exchange through shared memory
            float wmax[kDecQ];
#pragma unroll
            for (int q = 0; q < kDecQ; ++q) {
                int i = int(v[q]);
                i ^= (i >> 31) & 0x7fffffff;
                i = __reduce_max_sync(0xffffffffu, i);
                i ^= (i >> 31) & 0x7fffffff;
                wmax[q] = __int_as_float(i);
            }
            if (lane < kDecQ) {
                float mine = wmax[0];
#pragma unroll
                for (int q = 1; q < kDecQ; ++q) mine = lane == q ? wmax[q] : mine;
                pipe.mx[j & 1][warp][lane] = mine;
            }
            __syncwarp();
            if (lane == 0) rz::BarrierArrive::execute(&pipe.mx_bar[j & 1]);
            if (!(ok = wait_or_report(&pipe.mx_bar[j & 1], uint32_t((j >> 1) & 1), rz::kBarOther))) break;
            float factor[kDecQ];
            bool any_grow = false;
#pragma unroll
            for (int q4 = 0; q4 < kDecQ; q4 += 4) {
                const float4 a = *reinterpret_cast<const float4*>(&pipe.mx[j & 1][0][q4]);
                const float4 b = *reinterpret_cast<const float4*>(&pipe.mx[j & 1][1][q4]);
                const float4 d = *reinterpret_cast<const float4*>(&pipe.mx[j & 1][2][q4]);
                const float4 e = *reinterpret_cast<const float4*>(&pipe.mx[j & 1][3][q4]);
                const float m4[4] = {fmaxf(fmaxf(a.x, b.x), fmaxf(d.x, e.x)), fmaxf(fmaxf(a.y, b.y), fmaxf(d.y, e.y)),
                                     fmaxf(fmaxf(a.z, b.z), fmaxf(d.z, e.z)), fmaxf(fmaxf(a.w, b.w), fmaxf(d.w, e.w))};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int q = q4 + i;
                    factor[q] = 1.0f;
                    if (j == 0) {
                        ref[q] = (m4[i] == -INFINITY) ? 0.0f : m4[i];
                    } else if ((m4[i] - ref[q]) * c_of(q) > kRescaleThreshold) {      // the same decision in all 128 threads
                        factor[q] = rz::exp2_approx((ref[q] - m4[i]) * c_of(q));
                        ref[q] = m4[i];
                        l[q] *= factor[q];
                        any_grow = true;
                    }
                }
            }
            if (any_grow) {
                // O^T (lane = head-dim column, 16 query columns) is rescaled in place once the P.V of step j - 1 is complete
                if (!(ok = wait_or_report(&pipe.pv_done[(j - 1) & 1], uint32_t(((j - 1) >> 1) & 1), rz::kBarOther))) break;
                rz::Tcgen05FenceAfter::execute();
                uint32_t o[kDecQ];
                rz::TmemLoad32x16::execute(tO + lane_addr, o);
                rz::TmemLoadWait::execute(o);
#pragma unroll
                for (int q = 0; q < kDecQ; ++q) o[q] = __float_as_uint(__uint_as_float(o[q]) * factor[q]);
                rz::TmemStore32x16::execute(tO + lane_addr, o);
                rz::TmemStoreWait::execute();
            }
            // P^T buffer j & 1 was last read by the P.V of step j - 2
            if (j >= 2 && !(ok = wait_or_report(&pipe.pv_done[j & 1], uint32_t(((j >> 1) - 1) & 1), rz::kBarOther))) break;
            // P^T[q][key] = exp2(s c - ref c) as bf16 (E4M3): row q of a K-major 128-byte-swizzled tile, 64 (128) keys per
            // 128-byte span, 8 (16) keys per 16-byte chunk
            uint8_t* pbase = kFp8 ? sP + (j & 1) * kDecPBytes + (t & 15) : sP + (j & 1) * kDecPBytes + (t >> 6) * (kDecQ * 128) + (t & 7) * 2;
            const int chunk = kFp8 ? t >> 4 : (t & 63) >> 3;
#pragma unroll
            for (int q = 0; q < kDecQ; ++q) {
                const float e = rz::exp2_approx(fmaf(__uint_as_float(v[q]), c_of(q), -ref[q] * c_of(q)));
                l[q] += e;
                uint8_t* dst = pbase + q * 128 + ((chunk ^ (q & 7)) << 4);
                if constexpr (kFp8) *dst = uint8_t(rz::PackE4m3x4::execute(e, e, e, e) & 0xffu);
                else *reinterpret_cast<__nv_bfloat16*>(dst) = __float2bfloat16_rn(e);
            }
            rz::AsyncProxyFence::execute();
            rz::Tcgen05FenceBefore::execute();
            __syncwarp();
            if (lane == 0) rz::BarrierArrive::execute(&pipe.p_full[j & 1]);
        }
        // ---- partial result of this KV share: O^T to part_o (row = query, 128 consecutive floats per row), row sums
        //      reduced over the 128 threads, (reference in log2 units, sum) per row to part_ml ----
        const long long row0 = ((long long)blockIdx.z * p.num_heads + head_idx) * p.rows;
        if (p.direct) {
            // one KV share: the normalised rows and their LSE leave directly (row = bh * rows + q of the call's O and LSE)
            const long long orow0 = (long long)bh * p.rows;
            uint32_t o[kDecQ];
#pragma unroll
            for (int q = 0; q < kDecQ; ++q) o[q] = 0u;
            if (ok && n > 0) {
                ok = wait_or_report(&pipe.pv_done[(n - 1) & 1], uint32_t(((n - 1) >> 1) & 1), rz::kBarOther);
                if (ok) {
                    rz::Tcgen05FenceAfter::execute();
                    rz::TmemLoad32x16::execute(tO + lane_addr, o);
                    rz::TmemLoadWait::execute(o);
                }
            }
            if (ok) {
#pragma unroll
                for (int q = 0; q < kDecQ; ++q) {
                    float sum = l[q];
#pragma unroll
                    for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
                    l[q] = sum;
                }
                if (lane < kDecQ) {
                    float mine = l[0];
#pragma unroll
                    for (int q = 1; q < kDecQ; ++q) mine = lane == q ? l[q] : mine;
                    pipe.lsum[warp][lane] = mine;
                }
                __syncwarp();
                if (lane == 0) rz::BarrierArrive::execute(&pipe.l_bar);
                ok = wait_or_report(&pipe.l_bar, 0, rz::kBarOther);
            }
            if (ok) {
#pragma unroll
                for (int q4 = 0; q4 < kDecQ; q4 += 4) {
                    const float4 a = *reinterpret_cast<const float4*>(&pipe.lsum[0][q4]);
                    const float4 b = *reinterpret_cast<const float4*>(&pipe.lsum[1][q4]);
                    const float4 d = *reinterpret_cast<const float4*>(&pipe.lsum[2][q4]);
                    const float4 e = *reinterpret_cast<const float4*>(&pipe.lsum[3][q4]);
                    const float s4[4] = {(a.x + b.x) + (d.x + e.x), (a.y + b.y) + (d.y + e.y), (a.z + b.z) + (d.z + e.z), (a.w + b.w) + (d.w + e.w)};
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int q = q4 + i;
                        if (q < p.rows) {
                            // a row that sees no key: zeros and LSE = -inf, as the combine kernel leaves them
                            const float inv = s4[i] > 0.0f ? out_scale / s4[i] : 0.0f;
                            p.O[(orow0 + q) * kHeadDim + t] = __float2bfloat16_rn(__uint_as_float(o[q]) * inv);
                            if (p.LSE && t == q) p.LSE[orow0 + q] = s4[i] > 0.0f ? (ref[q] * c_of(q) + log2f(s4[i])) * kLn2 : -INFINITY;
                        }
                    }
                }
            }
        } else if (ok && n > 0) {
            ok = wait_or_report(&pipe.pv_done[(n - 1) & 1], uint32_t(((n - 1) >> 1) & 1), rz::kBarOther);
            if (ok) {
                rz::Tcgen05FenceAfter::execute();
                uint32_t o[kDecQ];
                rz::TmemLoad32x16::execute(tO + lane_addr, o);
                rz::TmemLoadWait::execute(o);
#pragma unroll
                for (int q = 0; q < kDecQ; ++q)
                    if (q < p.rows) p.part_o[(row0 + q) * kHeadDim + t] = __uint_as_float(o[q]) * out_scale;
#pragma unroll
                for (int q = 0; q < kDecQ; ++q) {
                    float s = l[q];
#pragma unroll
                    for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
                    l[q] = s;
                }
                if (lane < kDecQ) {
                    float mine = l[0];
#pragma unroll
                    for (int q = 1; q < kDecQ; ++q) mine = lane == q ? l[q] : mine;
                    pipe.lsum[warp][lane] = mine;
                }
                __syncwarp();
                if (lane == 0) rz::BarrierArrive::execute(&pipe.l_bar);
                if (warp == 0) {
                    ok = wait_or_report(&pipe.l_bar, 0, rz::kBarOther);
                    if (ok && lane < p.rows && lane < kDecQ) {
                        float mine = ref[0] * c_of(0);
#pragma unroll
                        for (int q = 1; q < kDecQ; ++q) mine = lane == q ? ref[q] * c_of(q) : mine;
                        const float sum = (pipe.lsum[0][lane] + pipe.lsum[1][lane]) + (pipe.lsum[2][lane] + pipe.lsum[3][lane]);
                        p.part_ml[row0 + lane] = make_float2(mine, sum);
                    }
                }
            }
        } else if (ok && warp == 0 && lane < p.rows) {
            p.part_ml[row0 + lane] = make_float2(-INFINITY, 0.0f);      // no key of this share is visible: an empty partial result
        }
    }

    rz::Tcgen05FenceBefore::execute();
    __syncthreads();
    if (warp == 5) {
        rz::Tcgen05FenceAfter::execute();
        rz::TmemDealloc<1>::execute(tmem_base, 64);
    }
}

// bytes of scratch memory a split-KV call needs: fp32 accumulator and (m, l) per row and KV share
int64_t splitkv_scratch_bytes(int64_t heads, int64_t Sq, int64_t splits) {
    return splits <= 1 ? 0 : splits * heads * Sq * int64_t(kHeadDim * 4 + 8);
}

template <bool kFp8>
int launch_attn(const void* Q, const void* K, const void* V, const float* dq, const float* dk, const float* dv, void* O,
                float* LSE, int64_t B, int64_t Hq, int64_t Hkv, int64_t Sq, int64_t Skv, int64_t D, float scale, int causal,
                int64_t splits, void* scratch, int64_t scratch_bytes, int64_t bh_begin, int64_t bh_end, void* stream,
                uint32_t* status_dev, bool stack_gqa = false, bool kv_shard = false, int64_t kv_pos0 = 0, int64_t skv_total = 0) {
    using namespace axp_shim;
    if (!Q || !K || !V || !O || (kFp8 && (!dq || !dk || !dv))) return fail(AXP_ERR_BAD_ARG, "attn: null pointer argument");
    if (B <= 0 || Hq <= 0 || Hkv <= 0 || Sq <= 0 || Skv <= 0) return fail(AXP_ERR_BAD_ARG, "attn: B, Hq, Hkv and the sequence lengths must be positive");
    if (!kv_shard) skv_total = Skv;
    if (kv_shard && (kv_pos0 < 0 || kv_pos0 + Skv > skv_total))
        return fail(AXP_ERR_BAD_ARG, "attn: KV shard [%lld, %lld) outside the sequence of %lld keys", (long long)kv_pos0, (long long)(kv_pos0 + Skv), (long long)skv_total);
    if (causal && Sq > skv_total) return fail(AXP_ERR_BAD_ARG, "attn: causal mask with more queries (%lld) than keys (%lld)", (long long)Sq, (long long)skv_total);
    if (splits < 1 || splits > 256) return fail(AXP_ERR_BAD_ARG, "attn: splits=%lld outside [1,256]", (long long)splits);
    const int64_t S = Skv;
    if (Hq % Hkv != 0) return fail(AXP_ERR_BAD_ARG, "attn: Hq=%lld is not a multiple of Hkv=%lld", (long long)Hq, (long long)Hkv);
    if (D != kHeadDim) return fail(AXP_ERR_UNSUPPORTED, "attn: head dim %lld (only 128 is realised)", (long long)D);
    if (S % (kFp8 ? 16 : 8) != 0) return fail(AXP_ERR_BAD_ARG, "attn: S=%lld must be a multiple of %d", (long long)S, kFp8 ? 16 : 8);
    if (bh_begin < 0 || bh_end > B * Hq || bh_begin > bh_end)
        return fail(AXP_ERR_BAD_ARG, "attn: head range [%lld,%lld) outside [0,%lld)", (long long)bh_begin, (long long)bh_end, (long long)(B * Hq));
    if (B * Hq > INT32_MAX / 2 || S > (1 << 24) || Sq > (1 << 24)) return fail(AXP_ERR_UNSUPPORTED, "attn: extent too large");
    const int64_t need = kv_shard ? (bh_end - bh_begin) * Sq * int64_t(kHeadDim * 4 + 8) : splitkv_scratch_bytes(bh_end - bh_begin, Sq, splits);
    if (need > 0 && (!scratch || scratch_bytes < need || (reinterpret_cast<uintptr_t>(scratch) & 255u)))
        return fail(AXP_ERR_BAD_ARG, "attn: split-KV needs %lld bytes of 256-byte aligned scratch memory (%lld given)", (long long)need, (long long)scratch_bytes);
    if (!(scale > 0.0f)) return fail(AXP_ERR_BAD_ARG, "attn: scale must be positive");
    if (!aligned16(Q) || !aligned16(K) || !aligned16(V) || !aligned16(O)) return fail(AXP_ERR_BAD_ARG, "attn: base pointers must be 16-byte aligned");
    if (bh_begin == bh_end) return AXP_OK;

    // Few queries per head (decode): the query heads that share a KV head are consecutive in memory, so Q, O and LSE of
    // a GQA group are one [group * Sq, D] block.  The launch then treats the group as one head with group * Sq rows: the
    // K / V tiles are read and multiplied once per group instead of once per query head.
    const int64_t q_per_head = Sq;
    {
        const int64_t grp = Hq / Hkv;
        if (stack_gqa && grp > 1 && 2 * Sq <= kTileM && bh_begin % grp == 0 && bh_end % grp == 0) {
            Sq *= grp;
            Hq = Hkv;
            bh_begin /= grp;
            bh_end /= grp;
        }
    }

    DeviceInfo dev;
    if (int rc = current_device_info(&dev); rc != AXP_OK) return rc;

    const CUtensorMapDataType dt = kFp8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    const uint64_t row_bytes = uint64_t(kHeadDim) * AttnCfg<kFp8>::kElem;

    // Decode: calls with few query rows per KV head take the kernel with swapped operands: with several KV shares or as one
    // shard of a KV-sharded call it leaves partial results, with one share it writes O and LSE itself
    {
        const int dec_opt = option_slot(kOptAttnDecode).load(std::memory_order_relaxed);
        if (Sq <= kDecQ && dec_opt != 1) {
            const int64_t heads = bh_end - bh_begin;
            CUtensorMap tmQd, tmKd, tmVd;
            {
                const uint64_t dims[3] = {uint64_t(kHeadDim), uint64_t(Sq), uint64_t(B * Hq)};
                const uint64_t strides[2] = {row_bytes, row_bytes * uint64_t(Sq)};
                const uint32_t qbox[3] = {uint32_t(DecCfg<kFp8>::kSpanElems), uint32_t(kDecQ), 1u};
                if (int rc = make_tensor_map(&tmQd, dt, 3, Q, dims, strides, qbox); rc != AXP_OK) return rc;
            }
            {
                const uint64_t dims[3] = {uint64_t(kHeadDim), uint64_t(S), uint64_t(B * Hkv)};
                const uint64_t strides[2] = {row_bytes, row_bytes * uint64_t(S)};
                const uint32_t kbox[3] = {uint32_t(DecCfg<kFp8>::kSpanElems), uint32_t(kDecKeys), 1u};
                if (int rc = make_tensor_map(&tmKd, dt, 3, K, dims, strides, kbox); rc != AXP_OK) return rc;
                if (int rc = make_tensor_map(&tmVd, dt, 3, V, dims, strides, kbox); rc != AXP_OK) return rc;
            }
            DecodeParams d;
            d.part_o = static_cast<float*>(scratch);
            d.part_ml = reinterpret_cast<float2*>(static_cast<float*>(scratch) + splits * heads * Sq * kHeadDim);
            d.rows = int(Sq);
            d.q_per_head = int(q_per_head);
            d.Skv = int(Skv);
            d.Hq = int(Hq);
            d.Hkv = int(Hkv);
            d.causal = causal ? 1 : 0;
            d.causal_off = int(skv_total - q_per_head - kv_pos0);      // local key 0 is global key kv_pos0
            d.bh_begin = int(bh_begin);
            d.num_heads = int(heads);
            const int64_t tiles = (Skv + kDecKeys - 1) / kDecKeys;
            d.tiles_per_split = int((tiles + splits - 1) / splits);
            d.scale = scale;
            d.status = status_dev;
            d.dq = dq;
            d.dk = dk;
            d.dv = dv;
            d.direct = (splits == 1 && !kv_shard) ? 1 : 0;
            d.O = static_cast<__nv_bfloat16*>(O);
            d.LSE = LSE;
            constexpr int kDecSmem = DecCfg<kFp8>::kSmem;
            static thread_local int decode_attr_set_for_device = -1;      // one per instantiation of this function template
            if (decode_attr_set_for_device != dev.device) {
                AXP_CUDA_TRY(cudaFuncSetAttribute(attn_decode_kernel<kFp8>, cudaFuncAttributeMaxDynamicSharedMemorySize, kDecSmem));
                decode_attr_set_for_device = dev.device;
            }
            attn_decode_kernel<kFp8><<<dim3(unsigned(heads), 1u, unsigned(splits)), kDecThreads, kDecSmem, static_cast<cudaStream_t>(stream)>>>(tmQd, tmKd, tmVd, d);
            AXP_CUDA_TRY(cudaGetLastError());
            if (!kv_shard && !d.direct) {
                const long long rows = (long long)heads * Sq;
                attn_splitkv_combine_kernel<<<unsigned((rows + 7) / 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
                    d.part_o, d.part_ml, rows * kHeadDim, rows, static_cast<__nv_bfloat16*>(O), LSE, rows, int(splits), (long long)bh_begin * Sq);
                AXP_CUDA_TRY(cudaGetLastError());
            }
            return AXP_OK;
        }
    }
    // tuning option "attn.kv_tile": keys per KV tile, 0 = library default, 64 (bf16 only) or 128
    const int kv_opt = option_slot(kOptAttnKvTile).load(std::memory_order_relaxed);
    const int kv_tile = kFp8 ? 128 : (kv_opt == 64 || kv_opt == 128 ? kv_opt : kDefaultKvTileBf16);
    const uint32_t box[3] = {uint32_t(AttnCfg<kFp8>::kSubCols), uint32_t(kTileM), 1u};
    const uint32_t kv_box[3] = {uint32_t(AttnCfg<kFp8>::kSubCols), uint32_t(kv_tile), 1u};
    CUtensorMap tmQ, tmK, tmV, tmO;
    {
        const uint64_t dims[3] = {uint64_t(kHeadDim), uint64_t(Sq), uint64_t(B * Hq)};
        const uint64_t strides[2] = {row_bytes, row_bytes * uint64_t(Sq)};
        if (int rc = make_tensor_map(&tmQ, dt, 3, Q, dims, strides, box); rc != AXP_OK) return rc;
        // O is bf16 for both operand types: 64 columns (128 bytes) x 128 rows per store
        const uint64_t o_strides[2] = {uint64_t(kHeadDim) * 2, uint64_t(kHeadDim) * 2 * uint64_t(Sq)};
        const uint32_t o_box[3] = {64u, uint32_t(kTileM), 1u};
        if (int rc = make_tensor_map(&tmO, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, O, dims, o_strides, o_box); rc != AXP_OK) return rc;
    }
    {
        const uint64_t dims[3] = {uint64_t(kHeadDim), uint64_t(S), uint64_t(B * Hkv)};
        const uint64_t strides[2] = {row_bytes, row_bytes * uint64_t(S)};
        if (int rc = make_tensor_map(&tmK, dt, 3, K, dims, strides, kv_box); rc != AXP_OK) return rc;
        if (int rc = make_tensor_map(&tmV, dt, 3, V, dims, strides, kv_box); rc != AXP_OK) return rc;
    }

    AttnParams p;
    p.O = O;
    p.LSE = LSE;
    p.dq = dq;
    p.dk = dk;
    p.dv = dv;
    p.Sq = int(Sq);
    p.q_per_head = int(q_per_head);
    p.Skv = int(Skv);
    p.Hq = int(Hq);
    p.Hkv = int(Hkv);
    p.causal = causal ? 1 : 0;
    p.bh_begin = int(bh_begin);
    p.num_q_blocks = int((Sq + kQTiles * kTileM - 1) / (kQTiles * kTileM));
    p.scale = scale;
    p.status = status_dev;
#if defined(AXP_SM100_LATENCY_PROBES)
    p.debug = reinterpret_cast<unsigned long long*>(debug_pointer().load(std::memory_order_relaxed));
    p.experiment = option_slot(kOptGemmExperiment).load(std::memory_order_relaxed);
#endif
    // tuning option "attn.issuers": 0 = library default, 1 or 2 MMA-issuing threads
    const int iss_opt = option_slot(kOptAttnIssuers).load(std::memory_order_relaxed);
    {
        // option "attn.rescale": 0 library default, 1 = standard online softmax (advance on every new maximum), 2 = lazy (2^8)
        const int r = option_slot(kOptAttnRescale).load(std::memory_order_relaxed);
        p.rescale_thr = r == 1 ? 0.0f : r == 2 ? kRescaleThreshold : (kFp8 ? kDefaultRescaleFp8 : kRescaleThreshold);
    }
    p.two_issuers = (iss_opt == 1 || iss_opt == 2) ? int(iss_opt == 2) : 1;   // measured with two: bf16 +12 %, E4M3 +4 %

    const int64_t heads = bh_end - bh_begin;
    if (heads > 65535) return fail(AXP_ERR_UNSUPPORTED, "attn: more than 65535 heads in one call");
    // split-KV: every share is a whole number of KV tiles
    const int64_t kv_tiles = (Skv + kv_tile - 1) / kv_tile;
    p.splits = int(splits);
    p.partial = (splits > 1 || kv_shard) ? 1 : 0;
    // query position i (inside its head) sees keys at global positions <= i + (skv_total - q_per_head); local key 0 is global kv_pos0
    p.causal_off = int(skv_total - q_per_head - kv_pos0);
    p.tiles_per_split = int((kv_tiles + splits - 1) / splits);
    p.part_o = static_cast<float*>(scratch);
    p.part_ml = reinterpret_cast<float2*>(static_cast<float*>(scratch) + splits * heads * Sq * kHeadDim);
    p.num_heads = int(heads);
    if (int64_t(p.num_q_blocks) * heads > INT32_MAX) return fail(AXP_ERR_UNSUPPORTED, "attn: more than 2^31-1 query blocks in one call");
    dim3 grid(unsigned(p.num_q_blocks) * unsigned(heads), 1u, unsigned(splits));
    // tuning option "attn.exp_mode": 0 = library default, otherwise 1 + kExpMode of the kernel template
    const int opt = option_slot(kOptAttnPolyExp).load(std::memory_order_relaxed);
    const int mode = opt == 0 ? (kFp8 ? kDefaultExpModeFp8 : kDefaultExpModeBf16) : opt - 1;
    // tuning option "attn.p_operand": 0 = library default, 1 = P in tensor memory, 2 = P through shared memory (E4M3 only)
    const int p_opt = option_slot(kOptAttnPOperand).load(std::memory_order_relaxed);
    const bool p_smem = kFp8 && (p_opt == 0 ? kDefaultPSmemFp8 : p_opt == 2);
    static thread_local int attr_set_for_device[2][12] = {{-1, -1, -1, -1, -1, -1, -1, -1, -1, -1, -1, -1},
                                                          {-1, -1, -1, -1, -1, -1, -1, -1, -1, -1, -1, -1}};
    auto launch = [&](auto kernel, int smem_bytes, int slot) -> int {
        if (attr_set_for_device[kFp8][slot] != dev.device) {
            if (int rc = check_register_pool(kernel, kAttnThreads, 128 * 56 + 256 * 224, "attn"); rc != AXP_OK) return rc;
            AXP_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
            attr_set_for_device[kFp8][slot] = dev.device;
        }
        kernel<<<grid, kAttnThreads, smem_bytes, static_cast<cudaStream_t>(stream)>>>(tmQ, tmK, tmV, tmO, p);
        AXP_CUDA_TRY(cudaGetLastError());
        return AXP_OK;
    };
    auto dispatch = [&]() -> int {
    if constexpr (kFp8) {
        if (p_smem) {
            constexpr int kBytes = AttnCfg<true, true>::kSmem;
            switch (mode) {
                case 1: return launch(attn_fwd_kernel<true, 1, true, 128>, kBytes, 5);
                case 2: return launch(attn_fwd_kernel<true, 2, true, 128>, kBytes, 6);
                case 3: return launch(attn_fwd_kernel<true, 3, true, 128>, kBytes, 7);
                default: return launch(attn_fwd_kernel<true, 0, true, 128>, kBytes, 4);
            }
        }
    }
    if constexpr (!kFp8) {
        if (kv_tile == 64) {
            constexpr int kBytes = AttnCfg<false, false, 64>::kSmem;
            switch (mode) {
                case 1: return launch(attn_fwd_kernel<false, 1, false, 64>, kBytes, 9);
                case 2: return launch(attn_fwd_kernel<false, 2, false, 64>, kBytes, 10);
                case 3: return launch(attn_fwd_kernel<false, 3, false, 64>, kBytes, 11);
                default: return launch(attn_fwd_kernel<false, 0, false, 64>, kBytes, 8);
            }
        }
    }
    constexpr int kBytes = AttnCfg<kFp8, false>::kSmem;
    switch (mode) {
        case 1: return launch(attn_fwd_kernel<kFp8, 1, false, 128>, kBytes, 1);
        case 2: return launch(attn_fwd_kernel<kFp8, 2, false, 128>, kBytes, 2);
        case 3: return launch(attn_fwd_kernel<kFp8, 3, false, 128>, kBytes, 3);
        default: return launch(attn_fwd_kernel<kFp8, 0, false, 128>, kBytes, 0);
    }
    };
    if (int rc = dispatch(); rc != AXP_OK) return rc;
    if (splits > 1 && !kv_shard) {
        const long long rows = (long long)heads * Sq;
        attn_splitkv_combine_kernel<<<unsigned((rows + 7) / 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
            p.part_o, p.part_ml, rows * kHeadDim, rows, static_cast<__nv_bfloat16*>(O), LSE, rows, int(splits), (long long)bh_begin * Sq);
        AXP_CUDA_TRY(cudaGetLastError());
    }
    return AXP_OK;
}

}  // namespace

extern "C" int axp_sm100_attn_fwd_bf16(const void* Q, const void* K, const void* V, void* O, float* LSE, int64_t B,
                                       int64_t Hq, int64_t Hkv, int64_t S, int64_t D, float scale, int causal,
                                       int64_t bh_begin, int64_t bh_end, void* stream, uint32_t* status_dev) {
    axp_shim::NvtxRange nvtx_range("axp_sm100_attn_fwd_bf16");
    return launch_attn<false>(Q, K, V, nullptr, nullptr, nullptr, O, LSE, B, Hq, Hkv, S, S, D, scale, causal, 1, nullptr, 0,
                              bh_begin, bh_end, stream, status_dev);
}

extern "C" int64_t axp_sm100_attn_splitkv_scratch_bytes(int64_t heads, int64_t Sq, int64_t num_splits) {
    if (heads <= 0 || Sq <= 0 || num_splits < 1) return -1;
    return splitkv_scratch_bytes(heads, Sq, num_splits);
}

extern "C" int axp_sm100_attn_fwd_bf16_splitkv(const void* Q, const void* K, const void* V, void* O, float* LSE, int64_t B,
                                               int64_t Hq, int64_t Hkv, int64_t Sq, int64_t Skv, int64_t D, float scale,
                                               int causal, int64_t num_splits, void* scratch, int64_t scratch_bytes,
                                               int64_t bh_begin, int64_t bh_end, void* stream, uint32_t* status_dev) {
    axp_shim::NvtxRange nvtx_range("axp_sm100_attn_fwd_bf16_splitkv");
    return launch_attn<false>(Q, K, V, nullptr, nullptr, nullptr, O, LSE, B, Hq, Hkv, Sq, Skv, D, scale, causal, num_splits,
                              scratch, scratch_bytes, bh_begin, bh_end, stream, status_dev, /*stack_gqa=*/true);
}

extern "C" int64_t axp_sm100_attn_partial_bytes(int64_t heads, int64_t Sq) {
    if (heads <= 0 || Sq <= 0) return -1;
    return heads * Sq * int64_t(kHeadDim * 4 + 8);
}

extern "C" int axp_sm100_attn_fwd_bf16_kvshard(const void* Q, const void* K, const void* V, void* partial, int64_t partial_bytes,
                                               int64_t B, int64_t Hq, int64_t Hkv, int64_t Sq, int64_t Skv_local, int64_t kv_pos0,
                                               int64_t Skv_total, int64_t D, float scale, int causal, int64_t bh_begin,
                                               int64_t bh_end, void* stream, uint32_t* status_dev) {
    axp_shim::NvtxRange nvtx_range("axp_sm100_attn_fwd_bf16_kvshard");
    if (!partial) return axp_shim::fail(AXP_ERR_BAD_ARG, "attn kvshard: partial buffer is null");
    // O and LSE are not written by a KV-shard pass: the partial buffer stands in for the (non-null) output argument
    return launch_attn<false>(Q, K, V, nullptr, nullptr, nullptr, partial, nullptr, B, Hq, Hkv, Sq, Skv_local, D, scale, causal, 1, partial,
                              partial_bytes, bh_begin, bh_end, stream, status_dev, /*stack_gqa=*/true, /*kv_shard=*/true, kv_pos0, Skv_total);
}

extern "C" int axp_sm100_attn_fwd_fp8_kvshard(const void* Q, const void* K, const void* V, const float* q_descale, const float* k_descale,
                                              const float* v_descale, void* partial, int64_t partial_bytes, int64_t B, int64_t Hq,
                                              int64_t Hkv, int64_t Sq, int64_t Skv_local, int64_t kv_pos0, int64_t Skv_total, int64_t D,
                                              float scale, int causal, int64_t bh_begin, int64_t bh_end, void* stream,
                                              uint32_t* status_dev) {
    axp_shim::NvtxRange nvtx_range("axp_sm100_attn_fwd_fp8_kvshard");
    if (!partial) return axp_shim::fail(AXP_ERR_BAD_ARG, "attn kvshard: partial buffer is null");
    return launch_attn<true>(Q, K, V, q_descale, k_descale, v_descale, partial, nullptr, B, Hq, Hkv, Sq, Skv_local, D, scale, causal, 1,
                             partial, partial_bytes, bh_begin, bh_end, stream, status_dev, /*stack_gqa=*/true, /*kv_shard=*/true, kv_pos0,
                             Skv_total);
}

extern "C" int axp_sm100_attn_combine_partials(const void* partials, int64_t num_shares, int64_t share_stride_bytes, void* O, float* LSE,
                                               int64_t rows, void* stream) {
    axp_shim::NvtxRange nvtx_range("axp_sm100_attn_combine_partials");
    using namespace axp_shim;
    if (!partials || !O) return fail(AXP_ERR_BAD_ARG, "attn combine: null pointer argument");
    if (num_shares < 1 || num_shares > 4096 || rows <= 0) return fail(AXP_ERR_BAD_ARG, "attn combine: bad share or row count");
    const int64_t share_bytes = rows * int64_t(kHeadDim * 4 + 8);
    if (share_stride_bytes < share_bytes || share_stride_bytes % 16 != 0 || (reinterpret_cast<uintptr_t>(partials) & 15u) || !aligned16(O))
        return fail(AXP_ERR_BAD_ARG, "attn combine: shares of %lld bytes need a stride >= that, a multiple of 16, and 16-byte aligned bases", (long long)share_bytes);
    const float* po = static_cast<const float*>(partials);
    const float2* pml = reinterpret_cast<const float2*>(po + rows * kHeadDim);
    attn_splitkv_combine_kernel<<<unsigned((rows + 7) / 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        po, pml, share_stride_bytes / 4, share_stride_bytes / 8, static_cast<__nv_bfloat16*>(O), LSE, rows, int(num_shares), 0);
    AXP_CUDA_TRY(cudaGetLastError());
    return AXP_OK;
}

// Scratch memory of the allocation-free split-KV entry point: part of the module image, 256-byte aligned, shared by
// all calls on a device (such calls must not overlap on one device).
namespace {
constexpr int64_t kStaticScratchBytes = int64_t(16) << 20;      // 16 MiB: splits * heads * Sq <= 32263 rows
static __device__ __align__(256) unsigned char g_splitkv_static_scratch[kStaticScratchBytes];
}  // namespace

extern "C" int64_t axp_sm100_attn_splitkv_static_scratch_bytes(void) { return kStaticScratchBytes; }

extern "C" int axp_sm100_attn_fwd_bf16_splitkv_static(const void* Q, const void* K, const void* V, void* O, float* LSE,
                                                      int64_t B, int64_t Hq, int64_t Hkv, int64_t Sq, int64_t Skv, int64_t D,
                                                      float scale, int causal, int64_t num_splits, int64_t bh_begin,
                                                      int64_t bh_end, void* stream, uint32_t* status_dev) {
    axp_shim::NvtxRange nvtx_range("axp_sm100_attn_fwd_bf16_splitkv_static");
    using namespace axp_shim;
    if (num_splits < 1 || Sq <= 0 || bh_begin < 0 || bh_end < bh_begin)
        return fail(AXP_ERR_BAD_ARG, "attn split-KV (static scratch): bad split count, query length or head range");
    const int64_t need = splitkv_scratch_bytes(bh_end - bh_begin, Sq, num_splits);
    if (need > kStaticScratchBytes)
        return fail(AXP_ERR_BAD_ARG, "attn split-KV (static scratch): %lld bytes needed, the built-in scratch holds %lld", (long long)need,
                    (long long)kStaticScratchBytes);
    // address of the scratch array on the current device, looked up once per device
    constexpr int kMaxDevices = 64;
    static std::atomic<void*> scratch_of_device[kMaxDevices];
    int device = -1;
    AXP_CUDA_TRY(cudaGetDevice(&device));
    if (device < 0 || device >= kMaxDevices) return fail(AXP_ERR_UNSUPPORTED, "attn split-KV (static scratch): device ordinal %d", device);
    void* scratch = scratch_of_device[device].load(std::memory_order_acquire);
    if (!scratch) {
        AXP_CUDA_TRY(cudaGetSymbolAddress(&scratch, g_splitkv_static_scratch));
        if (!scratch) return fail(AXP_ERR_CUDA, "attn split-KV (static scratch): symbol address is null");
        scratch_of_device[device].store(scratch, std::memory_order_release);
    }
    return launch_attn<false>(Q, K, V, nullptr, nullptr, nullptr, O, LSE, B, Hq, Hkv, Sq, Skv, D, scale, causal, num_splits, scratch,
                              kStaticScratchBytes, bh_begin, bh_end, stream, status_dev, /*stack_gqa=*/true);
}

extern "C" int axp_sm100_attn_fwd_fp8_splitkv(const void* Q, const void* K, const void* V, const float* q_descale,
                                              const float* k_descale, const float* v_descale, void* O, float* LSE, int64_t B,
                                              int64_t Hq, int64_t Hkv, int64_t Sq, int64_t Skv, int64_t D, float scale, int causal,
                                              int64_t num_splits, void* scratch, int64_t scratch_bytes, int64_t bh_begin,
                                              int64_t bh_end, void* stream, uint32_t* status_dev) {
    axp_shim::NvtxRange nvtx_range("axp_sm100_attn_fwd_fp8_splitkv");
    return launch_attn<true>(Q, K, V, q_descale, k_descale, v_descale, O, LSE, B, Hq, Hkv, Sq, Skv, D, scale, causal, num_splits,
                             scratch, scratch_bytes, bh_begin, bh_end, stream, status_dev, /*stack_gqa=*/true);
}

extern "C" int axp_sm100_attn_fwd_fp8(const void* Q, const void* K, const void* V, const float* q_descale,
                                      const float* k_descale, const float* v_descale, void* O, float* LSE, int64_t B,
                                      int64_t Hq, int64_t Hkv, int64_t S, int64_t D, float scale, int causal,
                                      int64_t bh_begin, int64_t bh_end, void* stream, uint32_t* status_dev) {
    axp_shim::NvtxRange nvtx_range("axp_sm100_attn_fwd_fp8");
    return launch_attn<true>(Q, K, V, q_descale, k_descale, v_descale, O, LSE, B, Hq, Hkv, S, S, D, scale, causal, 1, nullptr, 0,
                             bh_begin, bh_end, stream, status_dev);
}
