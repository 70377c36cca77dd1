// sm100 (Blackwell, sm_100a) leaf realizations: the device code behind the L0
// atoms that the gemm / attention recipes compose on iro::cap::sm100.
//
// The reference project ships this header as an empty namespace
// (include/axp/realize/sm100.hpp:9-14) and registers nothing for sm100
// (include/axp/kits/sm100/registry.hpp:10-14).  Every struct below follows the
// reference's realization shape -- a stateless struct with a
// `__device__ static void execute(raw pointers / words ...)` member, cf. the sm90
// leaf code at include/axp/realize/sm90.hpp:159-236 (stage issue), :1105-1340
// (barriers), :676-702 (MMA from descriptors) -- but is written for the sm_100a
// instruction set: raw mbarrier PTX with bounded waits, single-destination TMA,
// tcgen05.mma with accumulators in tensor memory, tcgen05.ld/st for the epilogue.
//
// Rules kept throughout:
//   * no wait spins without a limit: every wait returns false after the limit
//     and the caller records a status word and unwinds;
//   * every TMA load writes the shared memory of exactly one CTA;
//   * one elected thread issues TMA and tcgen05.mma; no block-wide barrier sits
//     between a copy and its consumer.
#pragma once

#include <cstdint>
#include <cuda.h>

#if defined(__CUDACC__)
#define AXP_DEV __device__ __forceinline__
#else
#define AXP_DEV inline
#endif

namespace axp::realize::sm100 {

// ----------------------------------------------------------------------------
// Status word written by a kernel whose bounded wait ran out.  Bits [0,8) name
// the role that gave up, bits [8,16) the barrier family, bit 31 marks "error".
// ----------------------------------------------------------------------------
enum : uint32_t {
    kStatusOk = 0u,
    kStatusError = 0x80000000u,
    kRoleProducer = 1u,
    kRoleMma = 2u,
    kRoleEpilogue = 3u,
    kRoleSoftmax = 4u,
    kRoleCorrection = 5u,
    kBarFull = 1u << 8,
    kBarEmpty = 2u << 8,
    kBarTmemFull = 3u << 8,
    kBarTmemEmpty = 4u << 8,
    kBarOther = 5u << 8,
};

// Wait limit: the clock is sampled every 256 polls; a wait gives up after this
// many SM cycles (about one second at 1.9 GHz, far above any legitimate wait).
constexpr long long kWaitLimitCycles = 2000000000LL;

#if defined(__CUDACC__)

AXP_DEV uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

AXP_DEV uint32_t lane_id() {
    uint32_t l;
    asm volatile("mov.u32 %0, %%laneid;" : "=r"(l));
    return l;
}

// One lane of a converged warp returns true.
AXP_DEV bool elect_one() {
    uint32_t pred = 0;
    asm volatile(
        "{\n\t"
        ".reg .pred P;\n\t"
        "elect.sync _|P, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, P;\n\t"
        "}\n"
        : "=r"(pred));
    return pred != 0;
}

// ----------------------------------------------------------------------------
// mbarrier atoms (reference contract family: include/axp/protocol/sync/contracts.hpp,
// sm90 realization include/axp/realize/sm90.hpp:1105-1340 on cuda::barrier).
// ----------------------------------------------------------------------------
struct BarrierInit {
    AXP_DEV static void execute(uint64_t* bar, uint32_t expected) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(expected));
    }
};

// Makes barrier initialisation visible to the async proxy (TMA, tcgen05.commit).
struct BarrierInitFence {
    AXP_DEV static void execute() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
};

struct BarrierExpectTx {
    AXP_DEV static void execute(uint64_t* bar, uint32_t bytes) {
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                     : "memory");
    }
};

struct BarrierArrive {
    AXP_DEV static void execute(uint64_t* bar) {
        asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
    }
};

// Arrive on the same-offset barrier of another CTA of the cluster.
struct ClusterBarrierArrive {
    AXP_DEV static void execute(uint64_t* bar, uint32_t cta_rank) {
        asm volatile(
            "{\n\t"
            ".reg .b32 remote;\n\t"
            "mapa.shared::cluster.u32 remote, %0, %1;\n\t"
            "mbarrier.arrive.release.cluster.shared::cluster.b64 _, [remote];\n\t"
            "}\n" ::"r"(smem_u32(bar)),
            "r"(cta_rank)
            : "memory");
    }
};

// The same remote arrive without release ordering: for hand-overs that publish no generic-proxy memory (a
// tensor-memory stage whose reads have completed under tcgen05.wait::ld and fence::before_thread_sync).  The
// releasing form orders all earlier memory operations of the thread at cluster scope first, which costs
// several hundred nanoseconds per arrive.
struct ClusterBarrierArriveRelaxed {
    AXP_DEV static void execute(uint64_t* bar, uint32_t cta_rank) {
        asm volatile(
            "{\n\t"
            ".reg .b32 remote;\n\t"
            "mapa.shared::cluster.u32 remote, %0, %1;\n\t"
            "mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [remote];\n\t"
            "}\n" ::"r"(smem_u32(bar)),
            "r"(cta_rank)
            : "memory");
    }
};

// Non-blocking probe (the reference models it as BarrierTryWait writing a flag,
// include/axp/realize/sm90.hpp:1300-1322).
struct BarrierTryWait {
    AXP_DEV static bool execute(uint64_t* bar, uint32_t parity) {
        uint32_t ok;
        asm volatile(
            "{\n\t"
            ".reg .pred P;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, P;\n\t"
            "}\n"
            : "=r"(ok)
            : "r"(smem_u32(bar)), "r"(parity)
            : "memory");
        return ok != 0;
    }
};

// Bounded wait.  Returns true when the phase completed; false when the limit ran
// out or *abort became non-zero (another role of this CTA already gave up).
struct BarrierWait {
    AXP_DEV static bool execute(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag) {
        if (BarrierTryWait::execute(bar, parity)) return true;
        const long long t0 = clock64();
        uint32_t polls = 0;
        while (true) {
            if (BarrierTryWait::execute(bar, parity)) return true;
            if ((++polls & 0xffu) == 0u) {
                if (*abort_flag != 0u) return false;
                if (clock64() - t0 > kWaitLimitCycles) return false;
            }
        }
    }
};

// Non-suspending probe: returns at once (mbarrier.test_wait), for a single thread
// that should notice a phase change with the least delay.
struct BarrierTestWait {
    AXP_DEV static bool execute(uint64_t* bar, uint32_t parity) {
        uint32_t ok;
        asm volatile(
            "{\n\t"
            ".reg .pred P;\n\t"
            "mbarrier.test_wait.parity.shared::cta.b64 P, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, P;\n\t"
            "}\n"
            : "=r"(ok)
            : "r"(smem_u32(bar)), "r"(parity)
            : "memory");
        return ok != 0;
    }
};

// Bounded wait built on the non-suspending probe.
struct BarrierSpinWait {
    AXP_DEV static bool execute(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag) {
        if (BarrierTestWait::execute(bar, parity)) return true;
        const long long t0 = clock64();
        uint32_t polls = 0;
        while (true) {
            if (BarrierTestWait::execute(bar, parity)) return true;
            if ((++polls & 0x3ffu) == 0u) {
                if (*abort_flag != 0u) return false;
                if (clock64() - t0 > kWaitLimitCycles) return false;
            }
        }
    }
};

// ----------------------------------------------------------------------------
// TMA atoms (reference contracts include/axp/protocol/tma/contracts.hpp:96-185,
// sm90 realization include/axp/realize/sm90.hpp:443-512).  Coordinates are
// (innermost, outer...); the innermost coordinate times the element size must be
// a multiple of 16 bytes.
// ----------------------------------------------------------------------------
struct PrefetchTensorMap {
    AXP_DEV static void execute(const CUtensorMap* map) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
    }
};

struct BulkTmaCopy2D {
    AXP_DEV static void execute(const CUtensorMap* map, void* smem_dst, int c0, int c1, uint64_t* bar) {
        asm volatile(
            "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
            ::"r"(smem_u32(smem_dst)),
            "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
            : "memory");
    }
};

struct BulkTmaCopy3D {
    AXP_DEV static void execute(const CUtensorMap* map, void* smem_dst, int c0, int c1, int c2, uint64_t* bar) {
        asm volatile(
            "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], "
            "[%2];" ::"r"(smem_u32(smem_dst)),
            "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
            : "memory");
    }
};

// 2-D copy whose completion is signalled on the barrier of CTA `leader_rank` of
// the cluster (same smem offset); data lands in this CTA's shared memory.  Used by
// the CTA pair of a cta_group::2 MMA: each CTA loads its own operand halves and
// the issuing CTA's barrier collects both.
struct BulkTmaCopy2DPeerBarrier {
    AXP_DEV static void execute(const CUtensorMap* map, void* smem_dst, int c0, int c1, uint64_t* bar,
                                uint32_t leader_rank) {
        asm volatile(
            "{\n\t"
            ".reg .b32 rbar;\n\t"
            "mapa.shared::cluster.u32 rbar, %2, %5;\n\t"
            "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, "
            "%4}], [rbar];\n\t"
            "}\n" ::"r"(smem_u32(smem_dst)),
            "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(leader_rank)
            : "memory");
    }
};

struct BulkTmaStore2D {
    AXP_DEV static void execute(const CUtensorMap* map, const void* smem_src, int c0, int c1) {
        asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                         reinterpret_cast<uint64_t>(map)),
                     "r"(smem_u32(smem_src)), "r"(c0), "r"(c1)
                     : "memory");
    }
};

struct BulkTmaStore3D {
    AXP_DEV static void execute(const CUtensorMap* map, const void* smem_src, int c0, int c1, int c2) {
        asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(
                         reinterpret_cast<uint64_t>(map)),
                     "r"(smem_u32(smem_src)), "r"(c0), "r"(c1), "r"(c2)
                     : "memory");
    }
};

struct BulkStoreCommit {
    AXP_DEV static void execute() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
};

// Waits until at most N committed store groups still read their shared memory.
template <int N>
struct BulkStoreWaitRead {
    AXP_DEV static void execute() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }
};

template <int N>
struct BulkStoreWaitAll {
    AXP_DEV static void execute() { asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory"); }
};

// Orders generic-proxy shared-memory writes before async-proxy reads (TMA store,
// tcgen05.mma operand fetch).  The reference's TileFence marks the same edge.
struct AsyncProxyFence {
    AXP_DEV static void execute() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
};

// ----------------------------------------------------------------------------
// Tensor-memory atoms (reference vocabulary: space::tmem, res::tmem_region,
// TileToTmem / TmemToTile contracts include/axp/protocol/tmem/contracts.hpp:21-132;
// no realization exists upstream).
// ----------------------------------------------------------------------------
template <int CtaGroup>
struct TmemAlloc {
    // Executed by one whole warp; writes the base address to *slot (shared memory).
    AXP_DEV static void execute(uint32_t* slot, uint32_t ncols) {
        if constexpr (CtaGroup == 1) {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)),
                         "r"(ncols)
                         : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        } else {
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)),
                         "r"(ncols)
                         : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
        }
    }
};

template <int CtaGroup>
struct TmemDealloc {
    AXP_DEV static void execute(uint32_t taddr, uint32_t ncols) {
        if constexpr (CtaGroup == 1) {
            asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
        } else {
            asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
        }
    }
};

struct Tcgen05FenceBefore {
    AXP_DEV static void execute() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
};
struct Tcgen05FenceAfter {
    AXP_DEV static void execute() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
};

// Arrives on an mbarrier once all tcgen05.mma issued so far by this thread have
// completed (implies fence::before_thread_sync).
template <int CtaGroup>
struct Tcgen05Commit {
    AXP_DEV static void execute(uint64_t* bar) {
        if constexpr (CtaGroup == 1) {
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                             smem_u32(bar))
                         : "memory");
        } else {
            asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                             smem_u32(bar))
                         : "memory");
        }
    }
};

// cta_group::2 commit that arrives on the same-offset barrier of every CTA in
// cta_mask (a barrier signal, not a data copy).
struct Tcgen05CommitPair {
    AXP_DEV static void execute(uint64_t* bar, uint16_t cta_mask) {
        asm volatile(
            "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
                smem_u32(bar)),
            "h"(cta_mask)
            : "memory");
    }
};

// Shared-memory matrix descriptor for tcgen05.mma (64-bit):
//   [0,14)  start address >> 4          [16,30) leading byte offset >> 4
//   [32,46) stride byte offset >> 4     [46,48) version = 1
//   [49,52) base offset = 0             [61,64) swizzle: 0 none, 2 = 128 B, 4 = 64 B, 6 = 32 B
// (the sm90 analogue is MakeWgmmaSmemDesc*, include/axp/realize/sm90.hpp:1512-1708,
// with a different bit layout).
//
// K-major operand, 128-byte swizzle: rows of 128 bytes, 8-row groups 1024 bytes
// apart (stride offset), leading offset unused (1).  The tile base must be
// 1024-byte aligned; stepping along K inside the 128-byte row adds the byte
// offset to the start address.
struct MakeSmemDescKMajorSw128 {
    AXP_DEV static uint64_t execute(uint32_t smem_addr) {
        uint64_t d = 0;
        d |= uint64_t((smem_addr & 0x3ffffu) >> 4);
        d |= uint64_t(1) << 16;
        d |= uint64_t(1024 >> 4) << 32;
        d |= uint64_t(1) << 46;
        d |= uint64_t(2) << 61;
        return d;
    }
};

// MN-major operand (the contiguous direction is M or N), 128-byte swizzle: an
// atom is 8 K-rows of 128 bytes (64 16-bit or 128 8-bit elements along MN);
// `lbo_bytes` steps to the next 128-byte span along MN, `sbo_bytes` to the next
// group of 8 K-rows.
struct MakeSmemDescMnMajorSw128 {
    AXP_DEV static uint64_t execute(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
        uint64_t d = 0;
        d |= uint64_t((smem_addr & 0x3ffffu) >> 4);
        d |= uint64_t((lbo_bytes >> 4) & 0x3fffu) << 16;
        d |= uint64_t((sbo_bytes >> 4) & 0x3fffu) << 32;
        d |= uint64_t(1) << 46;
        d |= uint64_t(2) << 61;
        return d;
    }
};

// Instruction descriptor (32-bit) for kind::f16 / kind::f8f6f4, fp32 accumulate:
//   [4,6) D format (1 = f32)   [7,10) A format   [10,13) B format
//   [15] A MN-major   [16] B MN-major   [17,23) N >> 3   [24,29) M >> 4
// formats: kind::f16: 0 = f16, 1 = bf16;  kind::f8f6f4: 0 = e4m3, 1 = e5m2.
enum class OperandFormat : uint32_t { F16 = 0, BF16 = 1, E4M3 = 0, E5M2 = 1 };

constexpr uint32_t make_instr_desc(uint32_t a_fmt, uint32_t b_fmt, bool a_mn_major, bool b_mn_major, uint32_t m,
                                   uint32_t n) {
    return (1u << 4) | (a_fmt << 7) | (b_fmt << 10) | (uint32_t(a_mn_major) << 15) | (uint32_t(b_mn_major) << 16) |
           ((n >> 3) << 17) | ((m >> 4) << 24);
}

// D[tmem] (+)= A[smem desc] * B[smem desc].  Issued by ONE thread.  Kind16 selects
// kind::f16 (f16/bf16 operands, K = 16 per instruction); otherwise kind::f8f6f4
// (8-bit operands, K = 32).  The reference contract is Tcgen05Mma
// (include/axp/protocol/compute/contracts.hpp:302-415).
template <int CtaGroup, bool Kind16>
struct Tcgen05Mma {
    AXP_DEV static void execute(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
        if constexpr (CtaGroup == 1 && Kind16) {
            asm volatile(
                "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n" ::"r"(tmem_d),
                "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
                : "memory");
        } else if constexpr (CtaGroup == 1 && !Kind16) {
            asm volatile(
                "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}\n" ::"r"(tmem_d),
                "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
                : "memory");
        } else if constexpr (CtaGroup == 2 && Kind16) {
            asm volatile(
                "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}\n" ::"r"(tmem_d),
                "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
                : "memory");
        } else {
            asm volatile(
                "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}\n" ::"r"(tmem_d),
                "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
                : "memory");
        }
    }
};

// The same MMA with each shared-memory descriptor given as two 32-bit words.  The high
// word of a 128-byte-swizzle descriptor is a constant (kSw128DescHi); the low word is
// (address >> 4) | (leading offset >> 4) << 16, so stepping through a tile is one 32-bit
// add per operand in the issuing thread (whose instruction stream is the limit for
// small MMAs).
constexpr uint32_t kSw128DescHi = (1024u >> 4) | (1u << 14) | (2u << 29);   // stride 1024 B, version 1, 128 B swizzle
AXP_DEV uint32_t sw128_desc_lo(uint32_t smem_addr, uint32_t lbo_bytes) {
    return ((smem_addr & 0x3ffffu) >> 4) | ((lbo_bytes >> 4) << 16);
}

template <bool Kind16>
struct Tcgen05MmaLo {
    // D[tmem] (+)= A[smem] * B[smem], cta_group::1
    AXP_DEV static void execute(uint32_t tmem_d, uint32_t a_lo, uint32_t b_lo, uint32_t idesc, uint32_t accumulate) {
        if constexpr (Kind16) {
            asm volatile(
                "{\n\t.reg .b64 da, db;\n\t.reg .pred p;\n\t"
                "mov.b64 da, {%1, %3};\n\tmov.b64 db, {%2, %3};\n\tsetp.ne.b32 p, %5, 0;\n\t"
                "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n\t}\n" ::"r"(tmem_d),
                "r"(a_lo), "r"(b_lo), "r"(kSw128DescHi), "r"(idesc), "r"(accumulate)
                : "memory");
        } else {
            asm volatile(
                "{\n\t.reg .b64 da, db;\n\t.reg .pred p;\n\t"
                "mov.b64 da, {%1, %3};\n\tmov.b64 db, {%2, %3};\n\tsetp.ne.b32 p, %5, 0;\n\t"
                "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], da, db, %4, p;\n\t}\n" ::"r"(tmem_d),
                "r"(a_lo), "r"(b_lo), "r"(kSw128DescHi), "r"(idesc), "r"(accumulate)
                : "memory");
        }
    }
    // D[tmem] (+)= A[tmem] * B[smem]
    AXP_DEV static void execute_tmem_a(uint32_t tmem_d, uint32_t tmem_a, uint32_t b_lo, uint32_t idesc, uint32_t accumulate) {
        if constexpr (Kind16) {
            asm volatile(
                "{\n\t.reg .b64 db;\n\t.reg .pred p;\n\t"
                "mov.b64 db, {%2, %3};\n\tsetp.ne.b32 p, %5, 0;\n\t"
                "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n\t}\n" ::"r"(tmem_d),
                "r"(tmem_a), "r"(b_lo), "r"(kSw128DescHi), "r"(idesc), "r"(accumulate)
                : "memory");
        } else {
            asm volatile(
                "{\n\t.reg .b64 db;\n\t.reg .pred p;\n\t"
                "mov.b64 db, {%2, %3};\n\tsetp.ne.b32 p, %5, 0;\n\t"
                "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], [%1], db, %4, p;\n\t}\n" ::"r"(tmem_d),
                "r"(tmem_a), "r"(b_lo), "r"(kSw128DescHi), "r"(idesc), "r"(accumulate)
                : "memory");
        }
    }
};

// Variant whose A operand is read from tensor memory (used for P in attention).
template <bool Kind16>
struct Tcgen05MmaTmemA {
    AXP_DEV static void execute(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
        if constexpr (Kind16) {
            asm volatile(
                "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}\n" ::"r"(tmem_d),
                "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
                : "memory");
        } else {
            asm volatile(
                "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], [%1], %2, %3, p;\n\t}\n" ::"r"(tmem_d),
                "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
                : "memory");
        }
    }
};

// Tensor memory -> registers, 32 lanes x 32-bit, 32 consecutive columns: lane i of
// the warp reads TMEM lane (lane base of taddr + i), columns [col, col+32).  A warp
// may only touch the 32-lane quarter (warp id % 4).  The data is valid after
// TmemLoadWait.
struct TmemLoad32x32 {
    AXP_DEV static void execute(uint32_t taddr, uint32_t (&r)[32]) {
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
            "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
            "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
            : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
              "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
              "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]),
              "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]),
              "=r"(r[30]), "=r"(r[31])
            : "r"(taddr)
            : "memory");
    }
};

struct TmemLoad32x16 {
    AXP_DEV static void execute(uint32_t taddr, uint32_t (&r)[16]) {
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
            "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
            : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
              "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
            : "r"(taddr)
            : "memory");
    }
};

struct TmemLoadWait {
    AXP_DEV static void execute() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
    // Same wait, with the loaded registers threaded through it, so that no use of
    // them can be scheduled ahead of the wait.
    AXP_DEV static void execute(uint32_t (&r)[32]) {
        asm volatile("tcgen05.wait::ld.sync.aligned;"
                     : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                       "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]),
                       "+r"(r[15]), "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]),
                       "+r"(r[22]), "+r"(r[23]), "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]),
                       "+r"(r[29]), "+r"(r[30]), "+r"(r[31])
                     :
                     : "memory");
    }
    AXP_DEV static void execute(uint32_t (&r)[16]) {
        asm volatile("tcgen05.wait::ld.sync.aligned;"
                     : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                       "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15])
                     :
                     : "memory");
    }
};

// Registers -> tensor memory, same lane/column mapping as TmemLoad32x32.
struct TmemStore32x32 {
    AXP_DEV static void execute(uint32_t taddr, const uint32_t (&r)[32]) {
        asm volatile(
            "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
            "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
            "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
            "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
            "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]),
            "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]),
            "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
            : "memory");
    }
};

struct TmemStore32x16 {
    AXP_DEV static void execute(uint32_t taddr, const uint32_t (&r)[16]) {
        asm volatile(
            "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
            "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
            "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
            "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
            : "memory");
    }
};

struct TmemStore32x8 {
    AXP_DEV static void execute(uint32_t taddr, const uint32_t (&r)[8]) {
        asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(taddr), "r"(r[0]),
                     "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
                     : "memory");
    }
};

struct TmemStoreWait {
    AXP_DEV static void execute() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
};

// ----------------------------------------------------------------------------
// Register budget moves between warpgroups (role specialisation; the reference's
// SpecializedOp gates roles per warpgroup, include/axp/level0/specialize.hpp:20-29).
// ----------------------------------------------------------------------------
template <int N>
struct RegDealloc {
    AXP_DEV static void execute() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N)); }
};
template <int N>
struct RegAlloc {
    AXP_DEV static void execute() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N)); }
};

// Named barrier over `threads` threads (reference: bar.sync id, threads at
// include/axp/realize/l0.hpp:1228).
struct NamedBarrierSync {
    AXP_DEV static void execute(uint32_t id, uint32_t threads) {
        asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
    }
};

// Cluster-wide arrive + wait (both CTAs of a pair), with release/acquire ordering.
struct ClusterSync {
    AXP_DEV static void execute() {
        asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    }
};

AXP_DEV uint32_t cluster_cta_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}

// ----------------------------------------------------------------------------
// Value atoms used by the epilogues.
// ----------------------------------------------------------------------------
// two fp32 -> packed bf16x2 (round to nearest even); `lo` lands in the low half.
struct PackBf16x2 {
    AXP_DEV static uint32_t execute(float lo, float hi) {
        uint32_t r;
        asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
        return r;
    }
};

// four fp32 -> four packed E4M3 bytes with saturation to +-448 (the fp8_saturate
// policy of include/axp/detail/conversion.hpp:83-95); a lands in the lowest byte.
struct PackE4m3x4 {
    AXP_DEV static uint32_t execute(float a, float b, float c, float d) {
        uint16_t lo, hi;
        asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(lo) : "f"(b), "f"(a));
        asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(hi) : "f"(d), "f"(c));
        return uint32_t(lo) | (uint32_t(hi) << 16);
    }
};

// Packed fp32 pairs in one 64-bit register: operands of the .f32x2 arithmetic of
// sm_100 (two fp32 operations per issue slot).
AXP_DEV unsigned long long pack_f32x2(float lo, float hi) {
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
AXP_DEV void unpack_f32x2(unsigned long long v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
AXP_DEV unsigned long long fma_f32x2(unsigned long long a, unsigned long long b, unsigned long long c) {
    unsigned long long d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
AXP_DEV unsigned long long add_f32x2(unsigned long long a, unsigned long long b) {
    unsigned long long d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
AXP_DEV unsigned long long mul_f32x2(unsigned long long a, unsigned long long b) {
    unsigned long long d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}

// exp2 of a packed pair on the FMA pipe (no SFU): round-to-nearest split x = n + f
// with the 1.5*2^23 trick, a degree-3 minimax polynomial for 2^f on [-0.5, 0.5]
// (relative error < 8e-5) and the integer n added into the exponent field.
// Inputs below -126 are clamped (the result is then ~1e-38, i.e. zero for softmax).
AXP_DEV void exp2_poly_f32x2(unsigned long long x2, float& e0, float& e1) {
    float x0, x1;
    unpack_f32x2(x2, x0, x1);
    x2 = pack_f32x2(fmaxf(x0, -126.0f), fmaxf(x1, -126.0f));
    const unsigned long long magic = pack_f32x2(12582912.0f, 12582912.0f);
    const unsigned long long neg_magic = pack_f32x2(-12582912.0f, -12582912.0f);
    const unsigned long long minus_one = pack_f32x2(-1.0f, -1.0f);
    const unsigned long long t2 = add_f32x2(x2, magic);             // low mantissa bits hold round(x)
    const unsigned long long n2 = add_f32x2(t2, neg_magic);         // round(x) as a float
    const unsigned long long f2 = fma_f32x2(n2, minus_one, x2);     // x - round(x)
    unsigned long long p2 = pack_f32x2(0.05508868396282196f, 0.05508868396282196f);
    p2 = fma_f32x2(p2, f2, pack_f32x2(0.24260404706001282f, 0.24260404706001282f));
    p2 = fma_f32x2(p2, f2, pack_f32x2(0.6932762265205383f, 0.6932762265205383f));
    p2 = fma_f32x2(p2, f2, pack_f32x2(0.9999289512634277f, 0.9999289512634277f));
    float p0, p1, t0, t1;
    unpack_f32x2(p2, p0, p1);
    unpack_f32x2(t2, t0, t1);
    e0 = __int_as_float(__float_as_int(p0) + (__float_as_int(t0) << 23));
    e1 = __int_as_float(__float_as_int(p1) + (__float_as_int(t1) << 23));
}

AXP_DEV float exp2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

AXP_DEV unsigned long long sub_f32x2(unsigned long long a, unsigned long long b) {
    unsigned long long d;
    asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}

// max(a, b, c) in one instruction (three-input max of sm_100).
AXP_DEV float max3_f32(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

// Sixteen softmax numerators e[i] = exp2(v[o16 + i] * c + neg) from scores held in registers, as eight packed
// pairs: one packed FMA per pair for the scale and shift, then per pair either two SFU ex2 or (pairs whose bit is
// set in kPolyMask) the degree-3 polynomial of exp2_poly_f32x2 on the FMA pipe, whose inputs are clamped at -126
// (masked scores are -inf).  The row sum is kept in two packed accumulators (four chains).
template <int kPolyMask>
AXP_DEV void exp2_block16(const uint32_t (&v)[32], int o16, unsigned long long c2, unsigned long long neg2,
                          unsigned long long& sum_a, unsigned long long& sum_b, float (&e)[16]) {
    const unsigned long long magic = pack_f32x2(12582912.0f, 12582912.0f);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const int o = o16 + 2 * k;
        unsigned long long x2 = fma_f32x2(pack_f32x2(__uint_as_float(v[o]), __uint_as_float(v[o + 1])), c2, neg2);
        float x0, x1;
        unpack_f32x2(x2, x0, x1);
        if ((kPolyMask >> k) & 1) {
            x2 = pack_f32x2(fmaxf(x0, -126.0f), fmaxf(x1, -126.0f));
            const unsigned long long t2 = add_f32x2(x2, magic);      // low mantissa bits hold round(x)
            const unsigned long long r2 = sub_f32x2(t2, magic);      // round(x) as a float
            const unsigned long long f2 = sub_f32x2(x2, r2);         // x - round(x) in [-0.5, 0.5]
            unsigned long long p2 = pack_f32x2(0.05508868396282196f, 0.05508868396282196f);
            p2 = fma_f32x2(p2, f2, pack_f32x2(0.24260404706001282f, 0.24260404706001282f));
            p2 = fma_f32x2(p2, f2, pack_f32x2(0.6932762265205383f, 0.6932762265205383f));
            p2 = fma_f32x2(p2, f2, pack_f32x2(0.9999289512634277f, 0.9999289512634277f));
            float p0, p1, t0, t1;
            unpack_f32x2(p2, p0, p1);
            unpack_f32x2(t2, t0, t1);
            e[2 * k] = __int_as_float(__float_as_int(p0) + (__float_as_int(t0) << 23));
            e[2 * k + 1] = __int_as_float(__float_as_int(p1) + (__float_as_int(t1) << 23));
        } else {
            e[2 * k] = exp2_approx(x0);
            e[2 * k + 1] = exp2_approx(x1);
        }
        if (k & 1) sum_b = add_f32x2(sum_b, pack_f32x2(e[2 * k], e[2 * k + 1]));
        else sum_a = add_f32x2(sum_a, pack_f32x2(e[2 * k], e[2 * k + 1]));
    }
}

// ----------------------------------------------------------------------------
// Leaves of the epilogue / softmax obligations (the device code the kernels call).
// ----------------------------------------------------------------------------
// ScalePromoteAccumulator: acc[i] = fma(s, partial[i], acc[i]) over the N partial sums a thread has read from tensor
// memory; s is the product of the operand scales of this K block (the reference's scale hook,
// include/axp/level3/gemm.hpp:104-116,1379-1382, applied to the fp32 partial sum instead of the operand tile).
struct ScalePromoteFma {
    template <int N>
    AXP_DEV static void execute(float* acc, const uint32_t (&partial)[N], float s) {
#pragma unroll
        for (int i = 0; i < N; ++i) acc[i] = fmaf(s, __uint_as_float(partial[i]), acc[i]);
    }
};

// Fused epilogues on eight consecutive fp32 accumulator columns, ending in packed bf16:
//   c_in != null : alpha * acc + beta * c_in as the reference's LinearCombinationVec evaluates it (MulAcc, MulC, Add:
//                  three fp32 operations, no contraction; include/axp/level3/gemm.hpp:187-208,221-234);
//   bias != null : act(acc + bias), act 0 = identity, 1 = SiLU x * sigmoid(x) with the Fast recipe's __expf
//                  (BiasActivationVec, gemm.hpp:159-219; SiLU include/axp/realize/l0.hpp:1955-1965);
//   neither      : plain cast.
struct BiasActFma {
    AXP_DEV static float activate(float x, float b, int act) {
        x += b;
        return act == 1 ? x / (1.0f + __expf(-x)) : x;
    }
    AXP_DEV static uint4 execute(const float (&f)[8], const float* bias, int act, const void* c_in = nullptr, float alpha = 1.0f,
                                 float beta = 0.0f) {
        float g[8];
        if (c_in) {
            const uint4 cv = *reinterpret_cast<const uint4*>(c_in);
            const uint32_t cw[4] = {cv.x, cv.y, cv.z, cv.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float c0 = __uint_as_float(cw[i] << 16), c1 = __uint_as_float(cw[i] & 0xffff0000u);
                g[2 * i] = __fadd_rn(__fmul_rn(alpha, f[2 * i]), __fmul_rn(beta, c0));
                g[2 * i + 1] = __fadd_rn(__fmul_rn(alpha, f[2 * i + 1]), __fmul_rn(beta, c1));
            }
        } else if (bias) {
            const float4 b0 = __ldg(reinterpret_cast<const float4*>(bias));
            const float4 b1 = __ldg(reinterpret_cast<const float4*>(bias) + 1);
            g[0] = activate(f[0], b0.x, act);
            g[1] = activate(f[1], b0.y, act);
            g[2] = activate(f[2], b0.z, act);
            g[3] = activate(f[3], b0.w, act);
            g[4] = activate(f[4], b1.x, act);
            g[5] = activate(f[5], b1.y, act);
            g[6] = activate(f[6], b1.z, act);
            g[7] = activate(f[7], b1.w, act);
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) g[i] = f[i];
        }
        uint4 o;
        o.x = PackBf16x2::execute(g[0], g[1]);
        o.y = PackBf16x2::execute(g[2], g[3]);
        o.z = PackBf16x2::execute(g[4], g[5]);
        o.w = PackBf16x2::execute(g[6], g[7]);
        return o;
    }
    // gated form: SiLU(gate) * up for two columns, packed
    AXP_DEV static uint32_t gated(float g0, float g1, float u0, float u1) {
        return PackBf16x2::execute(g0 / (1.0f + __expf(-g0)) * u0, g1 / (1.0f + __expf(-g1)) * u1);
    }
};

// StoreRowGlobal: eight packed bf16 columns (16 bytes) of one output row.
struct RowStoreVec16 {
    AXP_DEV static void execute(void* dst, uint4 v) { *reinterpret_cast<uint4*>(dst) = v; }
};

// RowSoftmaxStateUpdate: sixteen softmax numerators of one row and their running sums (see exp2_block16).
struct RowSoftmaxExp2 {
    template <int kPolyMask>
    AXP_DEV static void execute(const uint32_t (&v)[32], int o16, unsigned long long c2, unsigned long long neg2,
                                unsigned long long& sum_a, unsigned long long& sum_b, float (&e)[16]) {
        exp2_block16<kPolyMask>(v, o16, c2, neg2, sum_a, sum_b, e);
    }
};

#endif  // __CUDACC__

}  // namespace axp::realize::sm100
