#include "tile_iter_host.h"

#include "tile_iter.cuh"

namespace zx {

namespace {
struct HostParams {
  int causal, window_blocks, global_every;
  int n_q_tiles, n_kv_tiles;
  int q_tiles_per_chunk, kv_tiles_per_chunk;
  int q_chunk_pos[64];
  int kv_chunk_pos[64];
};
}  // namespace

int64_t tile_iter_mismatches(bool causal, int window_blocks, int global_every, const std::vector<int>& q_chunk_pos,
                             const std::vector<int>& kv_chunk_pos, int q_tiles_per_chunk, int kv_tiles_per_chunk) {
  HostParams p{};
  p.causal = causal; p.window_blocks = window_blocks; p.global_every = global_every;
  p.q_tiles_per_chunk = q_tiles_per_chunk; p.kv_tiles_per_chunk = kv_tiles_per_chunk;
  p.n_q_tiles = (int)q_chunk_pos.size() * q_tiles_per_chunk;
  p.n_kv_tiles = (int)kv_chunk_pos.size() * kv_tiles_per_chunk;
  if (q_chunk_pos.size() > 64 || kv_chunk_pos.size() > 64) return -1;
  for (size_t i = 0; i < q_chunk_pos.size(); ++i) p.q_chunk_pos[i] = q_chunk_pos[i];
  for (size_t i = 0; i < kv_chunk_pos.size(); ++i) p.kv_chunk_pos[i] = kv_chunk_pos[i];
  auto qpos = [&](int t) { return p.q_chunk_pos[t / p.q_tiles_per_chunk] + (t % p.q_tiles_per_chunk) * 128; };
  auto kpos = [&](int j) { return p.kv_chunk_pos[j / p.kv_tiles_per_chunk] + (j % p.kv_tiles_per_chunk) * 128; };
  int64_t bad = 0;
  for (int t = 0; t < p.n_q_tiles; ++t) {
    std::vector<int> want, got, got_cur;
    for (int j = 0; j < p.n_kv_tiles; ++j)
      if (ti_allowed(p, qpos(t), kpos(j))) want.push_back(j);
    for (int j = next_kv_tile(p, qpos(t), 0); j < p.n_kv_tiles; j = next_kv_tile(p, qpos(t), j + 1)) got.push_back(j);
    KvCursor cur;
    for (cur.init(p, qpos(t)); cur.j < p.n_kv_tiles; cur.seek(p, qpos(t), cur.j + 1)) {
      got_cur.push_back(cur.j);
      if (cur.kpos0 != kpos(cur.j)) ++bad;
    }
    if (got != want) ++bad;
    if (got_cur != want) ++bad;
    if (t + 1 < p.n_q_tiles && (t & 1) == 0) {        // the forward kernel's pairs
      PairWalk w;
      w.init(p, qpos(t), qpos(t + 1), true);
      std::vector<int> uni;
      for (int j = 0; j < p.n_kv_tiles; ++j)
        if (ti_allowed(p, qpos(t), kpos(j)) || ti_allowed(p, qpos(t + 1), kpos(j))) uni.push_back(j);
      size_t i = 0;
      while (w.advance(p, qpos(t), qpos(t + 1), true)) {
        if (i >= uni.size() || uni[i] != w.j) { ++bad; break; }
        if (w.need0 != ti_allowed(p, qpos(t), kpos(w.j)) || w.need1 != ti_allowed(p, qpos(t + 1), kpos(w.j))) ++bad;
        ++i;
      }
      if (i != uni.size()) ++bad;
    }
  }
  for (int j = 0; j < p.n_kv_tiles; ++j) {
    std::vector<int> want, got;
    for (int t = 0; t < p.n_q_tiles; ++t)
      if (ti_allowed(p, qpos(t), kpos(j))) want.push_back(t);
    for (int t = next_q_tile(p, kpos(j), 0); t < p.n_q_tiles; t = next_q_tile(p, kpos(j), t + 1)) got.push_back(t);
    if (got != want) ++bad;
  }
  return bad;
}

}  // namespace zx
