// Launch interface of the tcgen05 flash-attention kernels (head_dim 128, bf16, GQA).
//
// Positions are described by chunk tables rather than assumed contiguous: a Q (or KV) buffer of
// S tokens is `n_chunks` equal chunks, chunk c covering global positions
// [chunk_pos[c], chunk_pos[c] + chunk_len). That is exactly what a zigzag context-parallel
// shard looks like (two chunks), and a plain sequence is one chunk at position 0. Causal and
// block-sparse masks are evaluated from those global positions inside the kernel, tile by tile,
// so a masked-out 128x128 tile is never loaded or multiplied.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>
#include "../common/status.h"

namespace zx {

constexpr int kAttnMaxChunks = 8;

struct AttnMask {
  int causal = 1;
  int window_blocks = 0;  // > 0: keep only kv blocks with q_block - kv_block < window_blocks ...
  int global_every = 0;   // ... plus every kv block whose index is a multiple of this (0: none)
};

struct AttnLayout {
  int n_chunks = 1;
  int chunk_len = 0;
  int chunk_pos[kAttnMaxChunks] = {0};
};

struct AttnFwdArgs {
  // q: [B, Sq, Hq, 128] with token stride q_tok_stride (elements); k, v: [B, Skv, Hkv, 128] likewise.
  const void* q = nullptr;
  const void* k = nullptr;
  const void* v = nullptr;
  void* o = nullptr;      // [B, Sq, Hq, 128] contiguous bf16
  float* lse = nullptr;   // [B, Hq, Sq] natural-log sum-exp
  int B = 1, Hq = 0, Hkv = 0, Sq = 0, Skv = 0;
  int64_t q_tok_stride = 0, k_tok_stride = 0, v_tok_stride = 0;
  float scale = 0.f;
  AttnMask mask;
  AttnLayout q_layout, kv_layout;
  int merge_prev = 0;  // fold the result into the o/lse already present (ring step > 0)
  // Optional transfer fused into the kernel: one extra warp per CTA copies its slice of
  // [pull_src, pull_src + pull_bytes) (typically the next ring step's K/V in a peer GPU's memory)
  // into pull_dst (local staging) with plain P2P loads while the CTA computes.
  const void* pull_src = nullptr;
  void* pull_dst = nullptr;
  size_t pull_bytes = 0;
  Status* status = nullptr;
  cudaStream_t stream = nullptr;
};

void launch_attn_fwd(const AttnFwdArgs& args);

struct AttnBwdArgs {
  const void* q = nullptr;
  const void* k = nullptr;
  const void* v = nullptr;
  const void* o = nullptr;    // [B, Sq, Hq, 128]
  const void* d_o = nullptr;  // [B, Sq, Hq, 128]
  const float* lse = nullptr; // [B, Hq, Sq]
  float* delta = nullptr;     // [B, Hq, Sq] scratch: rowsum(dO * O), written by the pre-pass
  float* dq = nullptr;        // [B, Sq, Hq, 128] fp32, written (or accumulated when dq_accumulate)
  float* dk = nullptr;        // [B, Skv, Hkv, 128] fp32, red.add target, caller zeroes (may be a peer's buffer)
  float* dv = nullptr;        // [B, Skv, Hkv, 128] fp32, red.add target, caller zeroes (may be a peer's buffer)
  int B = 1, Hq = 0, Hkv = 0, Sq = 0, Skv = 0;
  int64_t q_tok_stride = 0, k_tok_stride = 0, v_tok_stride = 0;
  float scale = 0.f;
  AttnMask mask;
  AttnLayout q_layout, kv_layout;
  int compute_delta = 1;  // run the delta pre-pass (once per backward; later ring steps reuse it)
  int dq_accumulate = 0;  // add to the dq already present instead of overwriting it (ring step > 0)
  // Optional in-kernel timeline of the dQ kernel's first CTA: 64 iterations x 16 slots of SM clock
  // stamps (slots 0-5: compute thread 0 after each phase, 8-10: MMA warp). Null: no tracing.
  long long* trace = nullptr;
  const void* pull_src = nullptr;  // same fused peer pull as in the forward (done by the dK/dV kernel)
  void* pull_dst = nullptr;
  size_t pull_bytes = 0;
  Status* status = nullptr;
  cudaStream_t stream = nullptr;
};

void launch_attn_bwd(const AttnBwdArgs& args);

}  // namespace zx
