// Host model of the peer flag barrier (csrc/peer/peer_kernels.cu::peer_barrier_kernel): the same state
// machine on CPU threads and std::atomic, driven through randomised interleavings, so the protocol
// (per-pair epoch slots, release store, acquire poll, wrap-tolerant comparison, bounded wait) is checked
// without a GPU. Returns the number of protocol violations observed.
#pragma once
#include <cstdint>

namespace zx {

struct BarrierModelResult {
  int64_t violations;   // a rank left barrier k while some rank had not yet entered it, or saw stale data
  int64_t timeouts;     // bounded waits that expired
  int64_t rounds_done;  // barriers completed by every rank
};

// `ranks` threads run `rounds` barriers; before each barrier a rank publishes its round number in a plain
// (non-atomic) payload cell that every other rank reads right after the barrier. `start_epoch` lets the
// caller start just below the 32-bit wrap. `absent_rank` >= 0 never enters the barrier from
// `absent_from_round` on (its peers' waits must expire after `timeout_us`, not hang).
BarrierModelResult run_barrier_model(int ranks, int rounds, uint32_t start_epoch, uint64_t seed, int absent_rank,
                                     int absent_from_round, int64_t timeout_us);

}  // namespace zx
