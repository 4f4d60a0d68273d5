// Flash-attention forward for sm_100a (head_dim 128, bf16 in, fp32 softmax/accumulate).
//
// One CTA owns two adjacent 128-row Q tiles of one head and walks the KV buffer once:
//   warps 0-7    softmax of BOTH Q tiles, one tile at a time; warp (q, hf) owns 16 TMEM lanes (rows) and reads
//                them in the accumulator-fragment layout; S/P/O live in TMEM
//   warp 8       TMA producer: Q once, then K/V tiles through a 2-stage ring (plain per-CTA loads)
//   warps 9, 10  MMA issuers, one per Q tile: S_i = Q_i K^T (SS form) and O_i += P_i V (A = P read from
//                TMEM, issued in two halves so that it starts while the softmax finishes the row block)
//   warp 11      optional peer pull: copies this CTA's slice of the next ring step's K/V from the owning
//                GPU into local staging with plain P2P loads while the tiles compute
// The two Q tiles ping-pong so the tensor core has the other tile's MMAs to run during a softmax.
// TMEM (512 columns): S0 | S1 | O0 | O1, with the bf16 P_i written over the first half of S_i.
// O is only rescaled when a row's running max grew by more than 2^8 (the final 1/l makes the
// result exact either way). Causal / block-sparse masks come from global token positions, so the
// same kernel serves plain sequences, zigzag context-parallel shards and every ring step; with
// merge_prev it folds its result into the O/LSE left by the previous ring step.
#include "../common/ptx.cuh"
#include "../common/device_once.h"
#include "../common/tma_host.h"
#include "attn.h"
#include "tile_iter.cuh"

namespace zx {

namespace {

constexpr int HD = 128;
constexpr int BQ = 128;
constexpr int BKV = 128;
constexpr int TILE_BYTES = BQ * HD * 2;   // 32 KB
constexpr int HALF_BYTES = TILE_BYTES / 2; // one 64-wide d chunk: 128 rows x 128 B
constexpr int KV_STAGES = 2;
// Optional in-kernel timeline (compile with -DZX_FWD_TRACE): block 0 stamps the SM clock at the pipeline events
// of its first 256 KV tiles into a device array that zx_fwd_trace_read() copies out. Not part of normal builds.
#ifdef ZX_FWD_TRACE
__device__ long long g_fwd_trace[256 * 32];
#define ZX_TR(slot, iter) \
  do { if (blockIdx.x == 0 && lane == 0 && (iter) < 256u) g_fwd_trace[(iter) * 32 + (slot)] = clock64(); } while (0)
#else
#define ZX_TR(slot, iter) do { } while (0)
#endif

constexpr int TMA_WARP = 8, MMA_WARP0 = 9, MMA_WARP1 = 10, PULL_WARP = 11;
constexpr int NUM_THREADS = 12 * 32;
constexpr int TMEM_COLS = 512;
constexpr int SMEM_BYTES = 2 * TILE_BYTES + KV_STAGES * 2 * TILE_BYTES + 1024 + 256 + 2 * 2 * 128 * 4;
constexpr float NEG_BIG = -1.0e30f;
constexpr float RESCALE_THRESHOLD = 8.0f;

struct FwdParams {
  int B, Hq, Hkv, Sq, Skv;
  float scale_log2;
  int causal, window_blocks, global_every;
  int n_q_tiles, n_kv_tiles;
  int q_tiles_per_chunk, kv_tiles_per_chunk;
  int q_chunk_pos[kAttnMaxChunks];
  int kv_chunk_pos[kAttnMaxChunks];
  __nv_bfloat16* O;
  float* LSE;
  int merge_prev;
  const uint4* pull_src;
  uint4* pull_dst;
  size_t pull_nvec;
  Status* status;
};

__device__ __forceinline__ int q_tile_pos(const FwdParams& p, int t) {
  return p.q_chunk_pos[t / p.q_tiles_per_chunk] + (t % p.q_tiles_per_chunk) * BQ;
}
// warp-uniform bounded wait
__device__ __forceinline__ bool wait_warp(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  const bool ok = mbar_wait(bar, parity, abort_flag);
  return __all_sync(0xffffffffu, ok);
}

// Rare path of the softmax warps (a row's running maximum grew by more than the threshold): multiply this
// thread's entries of the output rows by their row's alpha in TMEM (fragment layout: registers 4k, 4k+1 belong
// to row a, 4k+2, 4k+3 to row b). Kept out of line so that its registers cost the hot loop nothing; the call's
// register saves only happen when the branch is taken.
__device__ __noinline__ void rescale_o_rows(uint32_t o_tmem, float alpha_a, float alpha_b) {
#pragma unroll 1
  for (int c = 0; c < 2; ++c) {
    uint32_t x[32];
    tmem_ld_16x256b_x8(o_tmem + c * 64, x);
    tmem_wait_ld();
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      x[4 * k] = __float_as_uint(__uint_as_float(x[4 * k]) * alpha_a);
      x[4 * k + 1] = __float_as_uint(__uint_as_float(x[4 * k + 1]) * alpha_a);
      x[4 * k + 2] = __float_as_uint(__uint_as_float(x[4 * k + 2]) * alpha_b);
      x[4 * k + 3] = __float_as_uint(__uint_as_float(x[4 * k + 3]) * alpha_b);
    }
    tmem_st_16x256b_x8(o_tmem + c * 64, x);
  }
  tmem_wait_st();
}

// Plain scan over the KV tiles with the position kept incrementally (no division per tile).
struct DenseWalk {
  int j, kpos0, left_in_chunk, c;
  __device__ __forceinline__ void init(const FwdParams& p) {
    j = 0; c = 0; kpos0 = p.kv_chunk_pos[0]; left_in_chunk = p.kv_tiles_per_chunk;
  }
  __device__ __forceinline__ void next(const FwdParams& p) {
    ++j;
    kpos0 += BKV;
    if (--left_in_chunk == 0) {
      ++c;
      left_in_chunk = p.kv_tiles_per_chunk;
      kpos0 = p.kv_chunk_pos[c < kAttnMaxChunks ? c : 0];
    }
  }
};
// tile_allowed() for the dense instantiation (no window).
__device__ __forceinline__ bool dense_allowed(const FwdParams& p, int qpos0, int kpos0) {
  return !(p.causal && kpos0 > qpos0);
}

#define ZX_FWD_SPARSE 0
#define ZX_FWD_KERNEL_NAME attn_fwd_kernel
#include "attn_fwd_kernel.inc"
#undef ZX_FWD_SPARSE
#undef ZX_FWD_KERNEL_NAME
#define ZX_FWD_SPARSE 1
#define ZX_FWD_KERNEL_NAME attn_fwd_sparse_kernel
#include "attn_fwd_kernel.inc"
#undef ZX_FWD_SPARSE
#undef ZX_FWD_KERNEL_NAME

CUtensorMap make_qkv_map(const void* base, int B, int S, int H, int64_t tok_stride) {
  uint64_t dims[4] = {(uint64_t)HD, (uint64_t)H, (uint64_t)S, (uint64_t)B};
  uint64_t strides[3] = {(uint64_t)HD * 2, (uint64_t)tok_stride * 2, (uint64_t)S * (uint64_t)tok_stride * 2};
  uint32_t box[4] = {64, 1, 128, 1};
  return make_tma_map(base, 2, 4, dims, strides, box, TmaSwizzle::B128);
}

}  // namespace

#ifdef ZX_FWD_TRACE
extern "C" int zx_fwd_trace_read(long long* host_dst) {
  return (int)cudaMemcpyFromSymbol(host_dst, g_fwd_trace, sizeof(long long) * 256 * 32);
}
#endif

void check_attn_common(int Hq, int Hkv, int Sq, int Skv, const AttnLayout& ql, const AttnLayout& kl) {
  if (Hq <= 0 || Hkv <= 0 || Hq % Hkv != 0) throw std::runtime_error("attention: Hq must be a multiple of Hkv");
  if (Sq % 128 != 0 || Skv % 128 != 0) throw std::runtime_error("attention: sequence lengths must be multiples of 128");
  if (ql.n_chunks < 1 || ql.n_chunks > kAttnMaxChunks || kl.n_chunks < 1 || kl.n_chunks > kAttnMaxChunks)
    throw std::runtime_error("attention: bad chunk count");
  if (ql.chunk_len * ql.n_chunks != Sq || kl.chunk_len * kl.n_chunks != Skv)
    throw std::runtime_error("attention: chunk table does not cover the buffer");
  if (ql.chunk_len % 128 != 0 || kl.chunk_len % 128 != 0)
    throw std::runtime_error("attention: chunk length must be a multiple of 128");
  for (int c = 0; c < ql.n_chunks; ++c)
    if (ql.chunk_pos[c] % 128 != 0) throw std::runtime_error("attention: chunk positions must be multiples of 128");
  for (int c = 0; c < kl.n_chunks; ++c)
    if (kl.chunk_pos[c] % 128 != 0) throw std::runtime_error("attention: chunk positions must be multiples of 128");
}

void launch_attn_fwd(const AttnFwdArgs& a) {
  check_attn_common(a.Hq, a.Hkv, a.Sq, a.Skv, a.q_layout, a.kv_layout);
  if (a.Sq == 0 || a.B == 0) return;
  CUtensorMap tmQ = make_qkv_map(a.q, a.B, a.Sq, a.Hq, a.q_tok_stride);
  CUtensorMap tmK = make_qkv_map(a.k, a.B, a.Skv, a.Hkv, a.k_tok_stride);
  CUtensorMap tmV = make_qkv_map(a.v, a.B, a.Skv, a.Hkv, a.v_tok_stride);
  FwdParams p;
  p.B = a.B; p.Hq = a.Hq; p.Hkv = a.Hkv; p.Sq = a.Sq; p.Skv = a.Skv;
  p.scale_log2 = a.scale * 1.4426950408889634f;
  p.causal = a.mask.causal; p.window_blocks = a.mask.window_blocks; p.global_every = a.mask.global_every;
  p.n_q_tiles = a.Sq / BQ;
  p.n_kv_tiles = a.Skv / BKV;
  p.q_tiles_per_chunk = a.q_layout.chunk_len / BQ;
  p.kv_tiles_per_chunk = a.kv_layout.chunk_len / BKV;
  for (int c = 0; c < kAttnMaxChunks; ++c) {
    p.q_chunk_pos[c] = c < a.q_layout.n_chunks ? a.q_layout.chunk_pos[c] : 0;
    p.kv_chunk_pos[c] = c < a.kv_layout.n_chunks ? a.kv_layout.chunk_pos[c] : 0;
  }
  p.O = (__nv_bfloat16*)a.o;
  p.LSE = a.lse;
  p.merge_prev = a.merge_prev;
  if (a.pull_bytes % 16 != 0) throw std::runtime_error("attn_fwd: pull size must be a multiple of 16 bytes");
  p.pull_src = (const uint4*)a.pull_src;
  p.pull_dst = (uint4*)a.pull_dst;
  p.pull_nvec = a.pull_src != nullptr ? a.pull_bytes / 16 : 0;
  p.status = a.status;
  static PerDeviceOnce once;
  bool& configured = once.current();
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(attn_fwd_sparse_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess)
      throw std::runtime_error(std::string("attn_fwd: cannot raise shared memory limit: ") + cudaGetErrorString(e));
    configured = true;
  }
  const int n_pairs = (p.n_q_tiles + 1) / 2;
  const int grid = n_pairs * a.Hq * a.B;
  if (p.window_blocks > 0) attn_fwd_sparse_kernel<<<grid, NUM_THREADS, SMEM_BYTES, a.stream>>>(tmQ, tmK, tmV, p);
  else attn_fwd_kernel<<<grid, NUM_THREADS, SMEM_BYTES, a.stream>>>(tmQ, tmK, tmV, p);
}

}  // namespace zx
