// Offline-optimal (Belady MIN) residency planning over byte-sized blocks.
#pragma once
#include <cstdint>
#include <vector>

namespace zxh {

struct BeladyResult {
  std::vector<uint8_t> hit;                    // per access: 1 if the block was resident
  std::vector<std::vector<int64_t>> evicted;   // per access: blocks evicted to make room
  std::vector<int64_t> next_use;               // per access: index of the next access to the same block, or -1
  int64_t hits = 0, misses = 0;
  int64_t bytes_loaded = 0, bytes_evicted = 0;
  int64_t peak_resident_bytes = 0;
  int64_t bypassed = 0;                        // blocks larger than the whole capacity (streamed, never resident)
};

// ids[i]: block touched by access i; size_of[id]: bytes of block id (ids are dense, 0..n-1).
BeladyResult belady_min(const std::vector<int64_t>& ids, const std::vector<int64_t>& size_of, int64_t capacity_bytes);

// Same trace under LRU, for comparison in reports and tests.
BeladyResult lru_trace(const std::vector<int64_t>& ids, const std::vector<int64_t>& size_of, int64_t capacity_bytes);

}  // namespace zxh
