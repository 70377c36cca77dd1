// Causal-mask index predicates shared by the attention kernels and the
// mask-tile entry point.  Integer work, identical on host and device.
//
// Reference: CausalMaskPred (include/axp/realize/l0.hpp:2563-2623):
//   valid(row, col) = (k_base + col) <= (q_base + row)           (l0.hpp:2613)
//   skip            = k_base > q_base + TileM - 1                (l0.hpp:2619)
#pragma once

#include <cstdint>

#if defined(__CUDACC__)
#define AXP_HD __host__ __device__ __forceinline__
#else
#define AXP_HD inline
#endif

namespace axp::realize::sm100 {

// key position k may be seen by query position q
AXP_HD bool causal_valid(long long q, long long k) { return k <= q; }

// the tile of keys starting at k_base lies wholly above the diagonal of the
// tile_m queries starting at q_base
AXP_HD bool causal_tile_skip(long long q_base, long long k_base, int tile_m) { return k_base > q_base + tile_m - 1; }

// number of KV tiles of tile_n keys that the tile_m queries starting at q_base
// can see under the causal mask (the remaining tiles are skipped whole)
AXP_HD int causal_kv_tiles(long long q_base, int tile_m, int tile_n, long long seq_len) {
    long long last = q_base + tile_m - 1;
    if (last > seq_len - 1) last = seq_len - 1;
    return int(last / tile_n) + 1;
}

// CausalMaskPredicate leaf: the element predicate and the whole-tile skip test.
struct CausalMaskPred {
    AXP_HD static bool execute(long long q, long long k) { return causal_valid(q, k); }
    AXP_HD static bool skip(long long q_base, long long k_base, int tile_m) { return causal_tile_skip(q_base, k_base, tile_m); }
};

}  // namespace axp::realize::sm100
