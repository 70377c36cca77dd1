// Intent vocabulary of the L4 patterns: portable wishes, no mechanism.
// Same names as the reference (include/axp/intent.hpp:7-31).
// Public surface restated from tribe-iro/iro-cuda-ax (MIT licence, Copyright (c) 2026 IRO; the notice is kept in
// THIRD_PARTY_NOTICES.md at the repository root).
#pragma once
#include <iro_cuda_ax_core.hpp>

namespace axp::intent {
namespace memory_pattern {
struct None {};
struct Optimized {};
struct Persistent {};
struct RingBuffered {};
}  // namespace memory_pattern
namespace load_mode {
struct Streaming {};
struct AsyncPrefetch {};
struct DeterministicLatency {};
}  // namespace load_mode
namespace schedule {
struct ProducerConsumer {};
struct Pipelined {};
struct BulkSynchronous {};
struct PersistentPipeline {};
struct DeterministicLatency {};
}  // namespace schedule
namespace tile_skip {
struct None {};
struct Causal {};
}  // namespace tile_skip
}  // namespace axp::intent
