// Host-side exhaustive check of the attention kernels' tile iteration (tile_iter.cuh) against a plain scan.
#pragma once
#include <cstdint>
#include <vector>

namespace zx {

// For every Q tile: the KV tiles found by next_kv_tile and by KvCursor must equal the tiles a plain scan with
// the mask predicate keeps; for every KV tile the same for next_q_tile; for every pair of adjacent Q tiles the
// PairWalk union and its need flags. Returns the number of mismatches (0 = the iteration is exact).
int64_t tile_iter_mismatches(bool causal, int window_blocks, int global_every, const std::vector<int>& q_chunk_pos,
                             const std::vector<int>& kv_chunk_pos, int q_tiles_per_chunk, int kv_tiles_per_chunk);

}  // namespace zx
