// Tile iteration for the attention kernels: "next KV tile at or after j that some Q tile may attend"
// and its mirror image over Q tiles, with jumps over runs of tiles that the mask provably excludes.
//
// Positions are piecewise contiguous (zigzag chunks), so inside one chunk the block index grows with
// the tile index. A jump only ever skips tiles for which tile_allowed() is false (tiles above the
// causal diagonal until the end of their chunk; tiles left of the window up to the next global block
// or the window's first block), and every candidate is still tested with tile_allowed(), so every
// role of a kernel sees the same sequence as a plain scan, at the cost of the kept tiles only.
// With a 4096-token window over 262,144 tokens a plain scan visits 2,048 tiles to find ~64.
#pragma once

// The functions are plain index arithmetic: compiled for the device by nvcc and, for the host-side
// exhaustive check against a brute-force scan (csrc/attn/tile_iter_host.cpp), by the host compiler.
#if defined(__CUDACC__)
#define ZX_TI_FN __host__ __device__ __forceinline__
#else
#define ZX_TI_FN inline
#endif

namespace zx {

template <class P>
ZX_TI_FN bool ti_allowed(const P& p, int qpos0, int kpos0) {
  if (p.causal && kpos0 > qpos0) return false;
  if (p.window_blocks > 0) {
    const int qb = qpos0 >> 7, kb = kpos0 >> 7;
    const int dist = qb >= kb ? qb - kb : kb - qb;
    const bool in_window = dist < p.window_blocks;
    const bool is_global = p.global_every > 0 && (kb % p.global_every) == 0;
    if (!in_window && !is_global) return false;
  }
  return true;
}

// Smallest KV tile j' >= j that Q tile position qpos0 may attend; n_kv_tiles if none.
template <class P>
ZX_TI_FN int next_kv_tile(const P& p, int qpos0, int j) {
  const int n = p.n_kv_tiles, per = p.kv_tiles_per_chunk;
  const int qb = qpos0 >> 7;
  while (j < n) {
    const int c = j / per;
    const int kpos0 = p.kv_chunk_pos[c] + (j - c * per) * 128;
    if (ti_allowed(p, qpos0, kpos0)) return j;
    const int chunk_end = (c + 1) * per;
    const int kb = kpos0 >> 7;
    int step = 1;
    if (p.causal && kb > qb) {
      step = chunk_end - j;                                   // the rest of this chunk is above the diagonal
    } else if (p.window_blocks > 0) {
      const int next_global = p.global_every > 0 ? (kb / p.global_every + 1) * p.global_every : (1 << 30);
      const int win_lo = qb - p.window_blocks + 1;
      if (kb < win_lo) step = (next_global < win_lo ? next_global : win_lo) - kb;       // left of the window
      else if (kb > qb + p.window_blocks - 1) step = next_global - kb;                  // right of it (non-causal)
    }
    if (step < 1) step = 1;
    j = (j + step < chunk_end) ? j + step : chunk_end;
  }
  return n;
}

// Cursor over the KV tiles one Q tile may attend: keeps the chunk of the current tile, so stepping costs
// no integer division (the forward kernel's MMA warp walks two of these, one per Q tile of its pair).
struct KvCursor {
  int j;          // current tile (n_kv_tiles when exhausted)
  int kpos0;      // its first position
  int c, base_j, end_j, chunk_pos;

  template <class P>
  ZX_TI_FN void init(const P& p, int qpos0) {
    c = 0; base_j = 0; end_j = p.kv_tiles_per_chunk < p.n_kv_tiles ? p.kv_tiles_per_chunk : p.n_kv_tiles;
    chunk_pos = p.kv_chunk_pos[0];
    seek(p, qpos0, 0);
  }
  // moves to the first allowed tile at or after `from` (from >= the current tile)
  template <class P>
  ZX_TI_FN void seek(const P& p, int qpos0, int from) {
    const int n = p.n_kv_tiles, qb = qpos0 >> 7;
    int jj = from;
    while (true) {
      while (jj >= end_j && end_j < n) {      // enter the chunk that holds jj
        ++c; base_j = end_j; end_j += p.kv_tiles_per_chunk; chunk_pos = p.kv_chunk_pos[c];
      }
      if (jj >= n) { j = n; kpos0 = 0; return; }
      const int kp = chunk_pos + (jj - base_j) * 128;
      if (ti_allowed(p, qpos0, kp)) { j = jj; kpos0 = kp; return; }
      const int kb = kp >> 7;
      int step = 1;
      if (p.causal && kb > qb) {
        step = end_j - jj;
      } else if (p.window_blocks > 0) {
        const int next_global = p.global_every > 0 ? (kb / p.global_every + 1) * p.global_every : (1 << 30);
        const int win_lo = qb - p.window_blocks + 1;
        if (kb < win_lo) step = (next_global < win_lo ? next_global : win_lo) - kb;
        else if (kb > qb + p.window_blocks - 1) step = next_global - kb;
      }
      if (step < 1) step = 1;
      jj = (jj + step < end_j) ? jj + step : end_j;
    }
  }
};

// The union of the KV tiles of the two Q tiles of a forward CTA, in order; need0 / need1 tell which of the
// two the current tile belongs to.
struct PairWalk {
  int j;
  bool need0, need1;
  KvCursor cur[2];
  template <class P>
  ZX_TI_FN void init(const P& p, int qpos_a, int qpos_b, bool has_b) {
    j = -1; need0 = need1 = false;
    cur[0].init(p, qpos_a);
    if (has_b) cur[1].init(p, qpos_b); else cur[1].j = p.n_kv_tiles;
  }
  template <class P>
  ZX_TI_FN bool advance(const P& p, int qpos_a, int qpos_b, bool has_b) {
    j = cur[0].j < cur[1].j ? cur[0].j : cur[1].j;
    if (j >= p.n_kv_tiles) return false;
    need0 = cur[0].j == j;
    need1 = cur[1].j == j;
    if (need0) cur[0].seek(p, qpos_a, j + 1);
    if (need1) cur[1].seek(p, qpos_b, j + 1);
    return true;
  }
};

// Smallest Q tile t' >= t that may attend KV tile position kpos0; n_q_tiles if none.
template <class P>
ZX_TI_FN int next_q_tile(const P& p, int kpos0, int t) {
  const int n = p.n_q_tiles, per = p.q_tiles_per_chunk;
  const int kb = kpos0 >> 7;
  const bool kv_global = p.window_blocks > 0 && p.global_every > 0 && (kb % p.global_every) == 0;
  while (t < n) {
    const int c = t / per;
    const int qpos0 = p.q_chunk_pos[c] + (t - c * per) * 128;
    if (ti_allowed(p, qpos0, kpos0)) return t;
    const int chunk_end = (c + 1) * per;
    const int qb = qpos0 >> 7;
    int step = 1;
    if (qb < kb) {
      // below the diagonal (causal) or left of the window: nothing is allowed before block
      // kb - window + 1 (non-causal window) or kb (causal)
      if (p.causal) step = kb - qb;
      else if (p.window_blocks > 0 && !kv_global && qb < kb - p.window_blocks + 1) step = kb - p.window_blocks + 1 - qb;
    } else if (p.window_blocks > 0 && !kv_global && qb > kb + p.window_blocks - 1) {
      step = chunk_end - t;                                   // past the window for the rest of this chunk
    }
    if (step < 1) step = 1;
    t = (t + step < chunk_end) ? t + step : chunk_end;
  }
  return n;
}

}  // namespace zx
