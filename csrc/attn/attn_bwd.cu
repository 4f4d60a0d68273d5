// Flash-attention backward for sm_100a (head_dim 128, bf16 in, fp32 accumulate), two kernels:
//
//  dkdv kernel  one CTA per (128-row KV tile, KV head): K and V stay in shared memory, the CTA
//               streams every (query head of the group, Q tile) pair that can see the tile and keeps
//               dK and dV in TMEM the whole time. It computes the *transposed* scores
//               S^T = K Q^T and dP^T = V dO^T so that P^T and dS^T land in TMEM with KV rows on the
//               lanes, which is exactly the A operand of dV += P^T dO and dK += dS^T Q.
//               The result is added to fp32 dK/dV with red.add (system scope): the destination may
//               be a peer GPU's buffer, which is how a ring step returns gradients to the KV owner.
//  dq kernel    one CTA per (Q tile, query head): S = Q K^T, dP = dO V^T, dQ += dS K with dS fed
//               from TMEM; deterministic, no atomics.
//
// In both kernels the MMA stream is staggered (S of the next tile is issued while the compute
// warps still turn dP into dS), so exponentials and tensor work overlap with a single softmax
// warpgroup. All waits are bounded.
#include "../common/ptx.cuh"
#include "../common/device_once.h"
#include "../common/tma_host.h"
#include "attn.h"
#include "tile_iter.cuh"

namespace zx {

void check_attn_common(int Hq, int Hkv, int Sq, int Skv, const AttnLayout& ql, const AttnLayout& kl);

namespace {

constexpr int HD = 128;
constexpr int BT = 128;                    // tile edge in tokens (both Q and KV)
constexpr int TILE_BYTES = BT * HD * 2;    // 32 KB
constexpr int HALF_BYTES = TILE_BYTES / 2; // one 64-wide d chunk
constexpr int NUM_THREADS = 352;           // dQ kernel: 8 compute warps (two warpgroups) + TMA warp + two MMA warps
constexpr int W_TMA = 8, W_MMA = 9, W_MMA_DQ = 10;   // dQ kernel roles (the dK/dV kernel has its own, below)
constexpr int N_COMPUTE = 256;             // compute threads
constexpr int TMEM_COLS = 512;
constexpr float LOG2E = 1.4426950408889634f;
// Every BWD_POLY_EVERY-th pair of exponentials can be evaluated as a polynomial on the FMA pipe instead of the
// special-function unit. Measured: these kernels are bound by instruction issue and by their dependency
// chain, not by that unit, and the polynomial's extra instructions cost as much as they save (29.1 ms with
// every second pair, 28.4 ms with none at S = 32768), so the default is none.
#ifndef BWD_POLY_EVERY
#define BWD_POLY_EVERY 1000000
#endif
#ifndef DQ_POLY_EVERY
#define DQ_POLY_EVERY BWD_POLY_EVERY
#endif
#ifndef DKDV_POLY_EVERY
#define DKDV_POLY_EVERY BWD_POLY_EVERY
#endif

struct BwdParams {
  int B, Hq, Hkv, Sq, Skv;
  float scale, scale_log2;
  int causal, window_blocks, global_every;
  int n_q_tiles, n_kv_tiles;
  int q_tiles_per_chunk, kv_tiles_per_chunk;
  int q_chunk_pos[kAttnMaxChunks];
  int kv_chunk_pos[kAttnMaxChunks];
  const float* lse;
  const float* delta;
  float* dq;
  float* dk;
  float* dv;
  int dq_accumulate;
  const uint4* pull_src;
  uint4* pull_dst;
  size_t pull_nvec;
  long long* trace;
  Status* status;
};

// Clock stamps of pipeline events into the caller's trace buffer (first CTA of each kernel). Compiled in only
// with -DZX_BWD_TRACE: the stamps cost issue slots in loops that are bound by instruction issue.
#ifdef ZX_BWD_TRACE
#define ZX_TRACE_DKDV(iter, slot)                                                     \
  do {                                                                                \
    if (p.trace != nullptr && blockIdx.x == 0 && (iter) < 64) p.trace[1024 + (iter) * 16 + (slot)] = clock64(); \
  } while (0)
#define ZX_TRACE(iter, slot)                                                          \
  do {                                                                                \
    if (p.trace != nullptr && blockIdx.x == 0 && (iter) < 64) p.trace[(iter) * 16 + (slot)] = clock64(); \
  } while (0)
#else
#define ZX_TRACE_DKDV(iter, slot) do { } while (0)
#define ZX_TRACE(iter, slot) do { } while (0)
#endif
#define ZX_TRACE_W(iter, k) do { } while (0)

__device__ __forceinline__ int q_tile_pos(const BwdParams& p, int t) {
  return p.q_chunk_pos[t / p.q_tiles_per_chunk] + (t % p.q_tiles_per_chunk) * BT;
}
__device__ __forceinline__ int kv_tile_pos(const BwdParams& p, int j) {
  return p.kv_chunk_pos[j / p.kv_tiles_per_chunk] + (j % p.kv_tiles_per_chunk) * BT;
}
// The Q tiles that may attend the KV tile at position kpos0, in order. The backward kernels are bound by
// instruction issue, and every role of a CTA walks this sequence once per item, so the dense instantiation
// keeps the position incrementally (no division, no search); windowed masks use the jumping search.
template <bool SPARSE>
struct QWalk {
  int t, qpos0, in_chunk, c;
  __device__ __forceinline__ void init() { t = -1; qpos0 = 0; in_chunk = 0; c = 0; }
  __device__ __forceinline__ bool next(const BwdParams& p, int kpos0) {
    if constexpr (SPARSE) {
      t = next_q_tile(p, kpos0, t + 1);
      if (t >= p.n_q_tiles) return false;
      qpos0 = q_tile_pos(p, t);
      return true;
    } else {
      for (;;) {
        if (++t >= p.n_q_tiles) return false;
        if (in_chunk == p.q_tiles_per_chunk) { ++c; in_chunk = 0; }
        qpos0 = p.q_chunk_pos[c] + in_chunk * BT;
        ++in_chunk;
        if (!(p.causal && kpos0 > qpos0)) return true;
      }
    }
  }
};
// The KV tiles the Q tile at position qpos0 may attend, in order.
template <bool SPARSE>
struct KvWalk {
  int j, kpos0, in_chunk, c;
  __device__ __forceinline__ void init() { j = -1; kpos0 = 0; in_chunk = 0; c = 0; }
  __device__ __forceinline__ bool next(const BwdParams& p, int qpos0) {
    if constexpr (SPARSE) {
      j = next_kv_tile(p, qpos0, j + 1);
      if (j >= p.n_kv_tiles) return false;
      kpos0 = kv_tile_pos(p, j);
      return true;
    } else {
      for (;;) {
        if (++j >= p.n_kv_tiles) return false;
        if (in_chunk == p.kv_tiles_per_chunk) { ++c; in_chunk = 0; }
        kpos0 = p.kv_chunk_pos[c] + in_chunk * BT;
        ++in_chunk;
        if (!(p.causal && kpos0 > qpos0)) return true;
      }
    }
  }
};

__device__ __forceinline__ bool wait_warp(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  const bool ok = mbar_wait(bar, parity, abort_flag);
  return __all_sync(0xffffffffu, ok);
}

__device__ __forceinline__ void red_add_v4_sys(float* addr, float a, float b, float c, float d) {
  asm volatile("red.relaxed.sys.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d)
               : "memory");
}

// Base descriptors of a [128 x 128] bf16 tile (built once per tile address) ...
__device__ __forceinline__ uint64_t base_kmajor(uint32_t tile_addr) { return make_smem_desc_sw128(tile_addr, 16, 1024); }
__device__ __forceinline__ uint64_t base_mnmajor(uint32_t tile_addr) {
  return make_smem_desc_sw128(tile_addr, HALF_BYTES, 1024);
}
// ------------------------------------------------------------------------------------------
// delta[b, h, s] = sum_d dO * O
// ------------------------------------------------------------------------------------------
__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ d_o,
                                  float* __restrict__ delta, int B, int S, int H) {
  const int warps_per_block = blockDim.x >> 5;
  const size_t row = (size_t)blockIdx.x * warps_per_block + (threadIdx.x >> 5);  // (b, s, h)
  const int lane = threadIdx.x & 31;
  if (row >= (size_t)B * S * H) return;
  const uint2 a = reinterpret_cast<const uint2*>(o + row * HD)[lane];
  const uint2 g = reinterpret_cast<const uint2*>(d_o + row * HD)[lane];
  const float2 a0 = unpack_bf16x2(a.x), a1 = unpack_bf16x2(a.y), g0 = unpack_bf16x2(g.x), g1 = unpack_bf16x2(g.y);
  float acc = a0.x * g0.x + a0.y * g0.y + a1.x * g1.x + a1.y * g1.y;
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if (lane == 0) {
    const int h = (int)(row % H);
    const size_t bs = row / H;
    const int s = (int)(bs % S);
    const int b = (int)(bs / S);
    delta[((size_t)b * H + h) * S + s] = acc;
  }
}

// ------------------------------------------------------------------------------------------
// dK / dV
// ------------------------------------------------------------------------------------------
// Q lives until dK of its item has been issued, dO only until dV: a 3-deep Q ring and a 2-deep dO
// ring free every slot a full iteration before its next tile is needed, which hides the TMA latency.
constexpr int Q_STAGES = 3, DO_STAGES = 2;
// Sixteen compute warps: four column groups of 32 queries times the four TMEM lane quarters. The
// exponential phase is bound by the special-function unit whatever the warp count; everything
// around it (TMEM round trips, barrier latency, the dS arithmetic) is per-warp serial time, and
// four warps per scheduler overlap it where two could not.
constexpr int KW_COMPUTE = 16, KW_TMA = 16, KW_MMA = 17, KW_PULL = 18;
constexpr int DKDV_THREADS = (KW_COMPUTE + 3) * 32;
// Tail of the dK/dV kernel's shared memory: alignment slack, barriers, and two buffers of 256
// per-query statistics (-lse * log2e for 128 queries, then -delta for the same 128).
constexpr int DKDV_ALIGN_SLACK = 768, DKDV_BAR_BYTES = 192, DKDV_STAT_BYTES = 2 * 256 * 4;
constexpr int DKDV_SMEM =
    2 * TILE_BYTES /*K,V*/ + (Q_STAGES + DO_STAGES) * TILE_BYTES + DKDV_ALIGN_SLACK + DKDV_BAR_BYTES + DKDV_STAT_BYTES;
static_assert(DKDV_SMEM <= 227 * 1024, "dK/dV kernel shared memory");

template <bool SPARSE>
__global__ void __launch_bounds__(DKDV_THREADS, 1)
attn_bwd_dkdv_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmdO,
                     const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV, BwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;
  uint8_t* sV = smem + TILE_BYTES;
  uint8_t* sQ = smem + 2 * TILE_BYTES;                 // [Q_STAGES]
  uint8_t* sdO = sQ + Q_STAGES * TILE_BYTES;           // [DO_STAGES]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sdO + DO_STAGES * TILE_BYTES);
  uint64_t* kv_full = bars;         // 1
  uint64_t* q_full = bars + 1;      // [3]
  uint64_t* q_empty = bars + 4;     // [3]
  uint64_t* do_full = bars + 7;     // [2]
  uint64_t* do_empty = bars + 9;    // [2]
  uint64_t* s_full = bars + 11;     // 1
  uint64_t* dp_full = bars + 12;    // 1
  uint64_t* p_ready = bars + 13;    // 1 (one arrival per compute warp)
  uint64_t* ds_ready = bars + 14;   // 1 (one arrival per compute warp)
  uint64_t* acc_done = bars + 15;   // 1
  uint64_t* drain_bar = bars + 16;  // 1
  uint64_t* stat_ready = bars + 17; // [2] (one arrival per publishing warp)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 19);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* stats = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(bars) + DKDV_BAR_BYTES);  // [2][256]
  if (smem - smem_raw > DKDV_ALIGN_SLACK) {  // same verdict in every thread
    if (threadIdx.x == 0) report(p.status, ZX_ERR_ARG, /*site=*/20, (int)(smem - smem_raw));
    return;
  }

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // Head-major: the CTAs in flight then share one or two heads' Q and dO tiles in L2 (measured 2 % faster than
  // spreading them over all heads). Inside a head, early KV tiles (most work under a causal mask) run first.
  int bid = blockIdx.x;
  const int j = bid % p.n_kv_tiles;
  bid /= p.n_kv_tiles;
  const int b = bid % p.B;
  const int hk = bid / p.B;
  const int G = p.Hq / p.Hkv;
  const int kpos0 = kv_tile_pos(p, j);

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int s = 0; s < Q_STAGES; ++s) {
      mbar_init(&q_full[s], 1);
      mbar_init(&q_empty[s], 1);
    }
    for (int s = 0; s < DO_STAGES; ++s) {
      mbar_init(&do_full[s], 1);
      mbar_init(&do_empty[s], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(dp_full, 1);
    mbar_init(p_ready, KW_COMPUTE);      // per-warp arrivals
    mbar_init(ds_ready, KW_COMPUTE);
    mbar_init(acc_done, 1);
    mbar_init(drain_bar, 1);
    mbar_init(&stat_ready[0], 8);
    mbar_init(&stat_ready[1], 8);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == KW_MMA) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // number of (head, q tile) items this CTA processes: identical in every role
  int n_items = 0;
  {
    QWalk<SPARSE> w;
    for (w.init(); w.next(p, kpos0);) ++n_items;
  }
  n_items *= G;

  if (warp == KW_PULL) warp_pull_slice(p.pull_src, p.pull_dst, p.pull_nvec, lane);

  if (n_items > 0 && warp < KW_PULL) {
    if (warp == KW_TMA) {
      // ------------------------------- TMA producer -------------------------------
      if (lane == 0) {
        tma_prefetch_desc(&tmQ);
        tma_prefetch_desc(&tmdO);
        mbar_expect_tx(kv_full, 2 * TILE_BYTES);
        tma_load_4d(sK, &tmK, kv_full, 0, hk, j * BT, b);
        tma_load_4d(sK + HALF_BYTES, &tmK, kv_full, 64, hk, j * BT, b);
        tma_load_4d(sV, &tmV, kv_full, 0, hk, j * BT, b);
        tma_load_4d(sV + HALF_BYTES, &tmV, kv_full, 64, hk, j * BT, b);
        uint32_t n = 0;
        bool ok = true;
        for (int g = 0; g < G && ok; ++g) {
          const int hq = hk * G + g;
          QWalk<SPARSE> w;
          for (w.init(); w.next(p, kpos0);) {
            const int t = w.t;
            const int qs = n % Q_STAGES, ds = n % DO_STAGES;
            if (!mbar_wait(&q_empty[qs], ((n / Q_STAGES) & 1) ^ 1, abort_flag)) { ok = false; break; }
            mbar_expect_tx(&q_full[qs], TILE_BYTES);
            tma_load_4d(sQ + qs * TILE_BYTES, &tmQ, &q_full[qs], 0, hq, t * BT, b);
            tma_load_4d(sQ + qs * TILE_BYTES + HALF_BYTES, &tmQ, &q_full[qs], 64, hq, t * BT, b);
            if (!mbar_wait(&do_empty[ds], ((n / DO_STAGES) & 1) ^ 1, abort_flag)) { ok = false; break; }
            mbar_expect_tx(&do_full[ds], TILE_BYTES);
            tma_load_4d(sdO + ds * TILE_BYTES, &tmdO, &do_full[ds], 0, hq, t * BT, b);
            tma_load_4d(sdO + ds * TILE_BYTES + HALF_BYTES, &tmdO, &do_full[ds], 64, hq, t * BT, b);
            ++n;
          }
        }
        if (!ok) {
          report(p.status, ZX_ERR_TIMEOUT, /*site=*/21, (int)n);
          const uint64_t t0 = globaltimer_ns();
          while (globaltimer_ns() - t0 < 2000000ull) {
          }
        }
      }
    } else if (warp == KW_MMA) {
      // ------------------------------- MMA issuer ---------------------------------
      {  // all 32 lanes run this loop; the instructions themselves are issued by one elected lane
        constexpr uint32_t idesc_kk = make_idesc(BT, BT, 1, 1, 0, 0);  // both operands K-major
        constexpr uint32_t idesc_tm = make_idesc(BT, HD, 1, 1, 0, 1);  // A from TMEM, B MN-major
        const uint32_t t_s = tmem_base, t_dp = tmem_base + 128, t_dv = tmem_base + 256, t_dk = tmem_base + 384;
        const uint64_t k_addr = base_kmajor(smem_u32(sK)), v_addr = base_kmajor(smem_u32(sV));
        const uint64_t q_k0 = base_kmajor(smem_u32(sQ)), do_k0 = base_kmajor(smem_u32(sdO));
        const uint64_t q_mn0 = base_mnmajor(smem_u32(sQ)), do_mn0 = base_mnmajor(smem_u32(sdO));
        bool ok = mbar_wait_w(kv_full, 0, abort_flag);
        ok = ok && mbar_wait_w(&q_full[0], 0, abort_flag);
        ok = ok && mbar_wait_w(&do_full[0], 0, abort_flag);
        tc_fence_after();
        if (ok) {
          umma_ss_k8_kmajor_w<HALF_BYTES / 16>(t_s, k_addr, q_k0, idesc_kk, 0u);
          umma_commit_w(s_full);
          umma_ss_k8_kmajor_w<HALF_BYTES / 16>(t_dp, v_addr, do_k0, idesc_kk, 0u);
          umma_commit_w(dp_full);
        }
        int n = 0;
        for (; n < n_items && ok; ++n) {
          const int qs = n % Q_STAGES, ds = n % DO_STAGES;
          const int qsn = (n + 1) % Q_STAGES, dsn = (n + 1) % DO_STAGES;
          const bool has_next = n + 1 < n_items;
          const uint64_t q_addr = desc_advance(q_mn0, (uint32_t)qs * TILE_BYTES);     // read transposed
          const uint64_t do_addr = desc_advance(do_mn0, (uint32_t)ds * TILE_BYTES);   // read transposed
          const uint64_t qn_addr = desc_advance(q_k0, (uint32_t)qsn * TILE_BYTES);
          const uint64_t don_addr = desc_advance(do_k0, (uint32_t)dsn * TILE_BYTES);
          // dV += P^T dO
          if (!mbar_wait_w(p_ready, n & 1, abort_flag)) { ok = false; break; }
          tc_fence_after();
          if (lane == 0) ZX_TRACE_DKDV(n, 8);
          umma_ts_k8_w<8, 32, 40, 64, 72, 96, 104>(t_dv, t_s, do_addr, idesc_tm, n > 0 ? 1u : 0u);
          umma_commit_w(&do_empty[ds]);   // dO(n) has now served dP^T(n) and dV(n)
          if (lane == 0) ZX_TRACE_DKDV(n, 9);
          if (has_next) {
            if (!mbar_wait_w(&q_full[qsn], ((n + 1) / Q_STAGES) & 1, abort_flag)) { ok = false; break; }
            tc_fence_after();
            if (lane == 0) ZX_TRACE_DKDV(n, 10);
            umma_ss_k8_kmajor_w<HALF_BYTES / 16>(t_s, k_addr, qn_addr, idesc_kk, 0u);
            umma_commit_w(s_full);
            if (lane == 0) ZX_TRACE_DKDV(n, 15);
          }
          // dK += dS^T Q
          if (!mbar_wait_w(ds_ready, n & 1, abort_flag)) { ok = false; break; }
          tc_fence_after();
          if (lane == 0) ZX_TRACE_DKDV(n, 11);
          umma_ts_k8_w<8, 32, 40, 64, 72, 96, 104>(t_dk, t_dp, q_addr, idesc_tm, n > 0 ? 1u : 0u);
          umma_commit_w(&q_empty[qs]);    // Q(n) has now served S^T(n) and dK(n)
          if (lane == 0) ZX_TRACE_DKDV(n, 12);
          if (has_next) {
            if (!mbar_wait_w(&do_full[dsn], ((n + 1) / DO_STAGES) & 1, abort_flag)) { ok = false; break; }
            tc_fence_after();
            if (lane == 0) ZX_TRACE_DKDV(n, 13);
            umma_ss_k8_kmajor_w<HALF_BYTES / 16>(t_dp, v_addr, don_addr, idesc_kk, 0u);
            umma_commit_w(dp_full);
          }
        }
        if (ok) umma_commit_w(acc_done);
        if (!ok) {
          if (lane == 0) report(p.status, ZX_ERR_TIMEOUT, /*site=*/22, n);
          umma_commit_w(drain_bar);
          const uint64_t t0 = globaltimer_ns();
          while (!mbar_try_wait(drain_bar, 0) && globaltimer_ns() - t0 < 50000000ull) {
          }
        }
      }
    } else {
      // ------------------------------- compute warps ------------------------------
      // Four column groups: group wg owns query columns [32 wg, 32 wg + 32) of every KV row.
      const int wg = warp >> 2;
      const int lq = warp & 3;                 // TMEM lane quarter
      const int r = lq * 32 + lane;            // KV row of this thread == TMEM lane
      const int col0 = wg * 32;
      const uint32_t lane_base = (uint32_t)(lq * 32) << 16;
      const uint32_t t_s = tmem_base + lane_base + col0, t_dp = tmem_base + lane_base + 128 + col0;
      const int my_kpos = kpos0 + r;
      uint32_t n = 0;
      bool ok = true;
      // Per-query statistics reach the math through shared memory, one item ahead: thread i of
      // the 256 fetches one value of the NEXT item (-lse * log2e for i < 128, -delta otherwise)
      // at the top of an iteration and publishes it at the bottom, so no global-load latency
      // sits between a TMEM read and its use. Buffer (n + 1) & 1 was last read in iteration
      // n - 1, and every thread finished that before dP^T(n) could be issued.
      const int ct = threadIdx.x;  // 0..255
      // this thread's statistic of item (g, t): -lse * log2e of query ct for ct < 128, else -delta of query ct - 128
      const float* stat_src = (ct < BT ? p.lse : p.delta) + ((size_t)b * p.Hq + (size_t)hk * G) * p.Sq + (ct & (BT - 1));
      const float stat_mul = ct < BT ? -LOG2E : -1.f;
      auto stat_fetch = [&](int g, int t) -> float {
        return stat_mul * __ldg(stat_src + (size_t)g * p.Sq + (size_t)t * BT);
      };
      QWalk<SPARSE> walk;
      auto next_item = [&](int& g) -> bool {   // advances walk (and g when a head's tiles are exhausted)
        for (;;) {
          if (walk.next(p, kpos0)) return true;
          walk.init();
          if (++g >= G) return false;
        }
      };
      int g = 0;
      walk.init();
      bool have = next_item(g);
      int t = walk.t, qpos0 = walk.qpos0;
      if (have && ct < 256) {
        stats[ct] = stat_fetch(g, t);
        mbar_arrive_warp(&stat_ready[0]);
      }
      while (have) {
        int gn = g;
        const bool have_next = next_item(gn);
        const int tn = walk.t, qposn = walk.qpos0;
        float pre = 0.f;
        if (have_next && ct < 256) pre = stat_fetch(gn, tn);
        const float* st = stats + (n & 1) * 256;
        if (!wait_warp(&stat_ready[n & 1], (n >> 1) & 1, abort_flag)) { ok = false; break; }
        ZX_TRACE_W(n, 7);
        if (!wait_warp(s_full, n & 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        if (threadIdx.x == 0) ZX_TRACE_DKDV(n, 0);
        ZX_TRACE_W(n, 0);
        uint32_t sr[32];
        tmem_ld_32x32b_x32(t_s, sr);
        tmem_wait_ld();
        ZX_TRACE_W(n, 1);
        const bool diag = p.causal && (kpos0 + BT - 1 > qpos0);
        const int qp = qpos0 + col0;   // column c is query qp + c; it sees this key iff my_kpos <= qp + c
        const float2 sl2 = make_float2(p.scale_log2, p.scale_log2);
        const float4* nl4 = reinterpret_cast<const float4*>(st + col0);   // uniform address: broadcast reads
        static_for<8>([&](auto idx4) {
          constexpr int c4 = decltype(idx4)::value;
          const float4 nl = nl4[c4];
          static_for<2>([&](auto idxh) {
            constexpr int h = decltype(idxh)::value;
            constexpr int c = 2 * c4 + h;
            const float2 x = __ffma2_rn(make_float2(__uint_as_float(sr[2 * c]), __uint_as_float(sr[2 * c + 1])), sl2,
                                        h == 0 ? make_float2(nl.x, nl.y) : make_float2(nl.z, nl.w));
            const float2 e = exp2_pair<c, DKDV_POLY_EVERY>(x);
            sr[2 * c] = __float_as_uint(e.x);
            sr[2 * c + 1] = __float_as_uint(e.y);
          });
        });
        if (diag) {   // only tiles on the diagonal pay for the per-element mask
#pragma unroll
          for (int c = 0; c < 32; ++c)
            if (my_kpos > qp + c) sr[c] = 0u;
        }
        ZX_TRACE_W(n, 2);
        {
          // bf16 P^T of this group goes over the first 16 of the 32 columns this thread just read
          uint32_t pk[16];
#pragma unroll
          for (int c = 0; c < 16; ++c) pk[c] = pack_bf16x2(__uint_as_float(sr[2 * c]), __uint_as_float(sr[2 * c + 1]));
          tmem_st_32x32b_x16(t_s, pk);
        }
        tmem_wait_st();
        if (threadIdx.x == 0) ZX_TRACE_DKDV(n, 2);
        ZX_TRACE_W(n, 3);
        tc_fence_before();
        mbar_arrive_warp(p_ready);
        if (!wait_warp(dp_full, n & 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        if (threadIdx.x == 0) ZX_TRACE_DKDV(n, 3);
        ZX_TRACE_W(n, 4);
        uint32_t dp[32];
        tmem_ld_32x32b_x32(t_dp, dp);
        tmem_wait_ld();
        ZX_TRACE_W(n, 5);
        {
          uint32_t dsp[16];
          const float4* nd4 = reinterpret_cast<const float4*>(st + BT + col0);
#pragma unroll
          for (int e4 = 0; e4 < 8; ++e4) {
            const float4 nd = nd4[e4];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              const int e = 2 * e4 + h;
              const float2 t2 = __fadd2_rn(make_float2(__uint_as_float(dp[2 * e]), __uint_as_float(dp[2 * e + 1])),
                                           h == 0 ? make_float2(nd.x, nd.y) : make_float2(nd.z, nd.w));
              const float2 d = __fmul2_rn(make_float2(__uint_as_float(sr[2 * e]), __uint_as_float(sr[2 * e + 1])), t2);
              dsp[e] = pack_bf16x2(d.x, d.y);
            }
          }
          tmem_st_32x32b_x16(t_dp, dsp);
        }
        tmem_wait_st();
        if (threadIdx.x == 0) ZX_TRACE_DKDV(n, 5);
        ZX_TRACE_W(n, 6);
        tc_fence_before();
        mbar_arrive_warp(ds_ready);
        if (have_next && ct < 256) {
          stats[((n + 1) & 1) * 256 + ct] = pre;
          mbar_arrive_warp(&stat_ready[(n + 1) & 1]);
        }
        g = gn;
        t = tn;
        qpos0 = qposn;
        have = have_next;
        ++n;
      }
      // epilogue: add dV and scale * dK into the (possibly remote) fp32 accumulators; each
      // column group drains its 32 columns of both accumulators
      if (ok) ok = wait_warp(acc_done, 0, abort_flag);
      tc_fence_after();
      if (ok && ZX_IN_BOUNDS(p.status, j * BT + r, p.Skv, 24)) {
        const size_t row_off = (((size_t)b * p.Skv + (size_t)j * BT + r) * p.Hkv + hk) * HD + col0;
        float* dv_row = p.dv + row_off;
        float* dk_row = p.dk + row_off;
        {
          uint32_t a[32];
          tmem_ld_32x32b_x32(tmem_base + lane_base + 256 + col0, a);
          tmem_wait_ld();
#pragma unroll
          for (int e = 0; e < 8; ++e)
            red_add_v4_sys(dv_row + e * 4, __uint_as_float(a[4 * e]), __uint_as_float(a[4 * e + 1]),
                           __uint_as_float(a[4 * e + 2]), __uint_as_float(a[4 * e + 3]));
        }
        {
          uint32_t a[32];
          tmem_ld_32x32b_x32(tmem_base + lane_base + 384 + col0, a);
          tmem_wait_ld();
#pragma unroll
          for (int e = 0; e < 8; ++e)
            red_add_v4_sys(dk_row + e * 4, __uint_as_float(a[4 * e]) * p.scale, __uint_as_float(a[4 * e + 1]) * p.scale,
                           __uint_as_float(a[4 * e + 2]) * p.scale, __uint_as_float(a[4 * e + 3]) * p.scale);
        }
      }
      if (!ok && lane == 0) report(p.status, ZX_ERR_TIMEOUT, /*site=*/23, (int)n);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == KW_MMA) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ------------------------------------------------------------------------------------------
// dQ
// ------------------------------------------------------------------------------------------
// K lives until dQ of its item has been issued, V only until dP: a 3-deep K ring and a 2-deep V
// ring free every slot a full iteration before its next tile is needed (hides the TMA latency).
constexpr int K_STAGES = 3, V_STAGES = 2;
constexpr int DQ_SMEM = 2 * TILE_BYTES /*Q,dO*/ + (K_STAGES + V_STAGES) * TILE_BYTES + 1024 + 256;   // barriers: 21 x 8 B

template <bool SPARSE>
__global__ void __launch_bounds__(NUM_THREADS, 1)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmdO,
                   const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV, BwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sdO = smem + TILE_BYTES;
  uint8_t* sK = smem + 2 * TILE_BYTES;            // [K_STAGES]
  uint8_t* sV = sK + K_STAGES * TILE_BYTES;       // [V_STAGES]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sV + V_STAGES * TILE_BYTES);
  uint64_t* qdo_full = bars;       // 1
  uint64_t* k_full = bars + 1;     // [3]
  uint64_t* k_empty = bars + 4;    // [3]
  uint64_t* v_full = bars + 7;     // [2]
  uint64_t* v_empty = bars + 9;    // [2]
  uint64_t* s_full = bars + 11;    // 1
  uint64_t* dp_full = bars + 12;   // 1
  uint64_t* s_read = bars + 13;    // 1 (one arrival per compute warp)
  uint64_t* ds_ready = bars + 14;  // 1 (one arrival per compute warp)
  uint64_t* acc_done = bars + 15;  // 1
  uint64_t* drain_bar = bars + 16; // [2]
  uint64_t* dp_free = bars + 18;   // [2] dQ of the item that used this dP buffer has finished reading it
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 20);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // Head-major, late Q tiles (most work) first inside a head: the CTAs in flight stream the same K and V.
  int bid = blockIdx.x;
  const int t = p.n_q_tiles - 1 - bid % p.n_q_tiles;
  bid /= p.n_q_tiles;
  const int b = bid % p.B;
  const int hq = bid / p.B;
  const int hk = hq / (p.Hq / p.Hkv);
  const int qpos0 = q_tile_pos(p, t);

  if (threadIdx.x == 0) {
    mbar_init(qdo_full, 1);
    for (int s = 0; s < K_STAGES; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
    }
    for (int s = 0; s < V_STAGES; ++s) {
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(dp_full, 1);
    mbar_init(s_read, N_COMPUTE / 32);    // per-warp arrivals
    mbar_init(ds_ready, N_COMPUTE / 32);
    mbar_init(acc_done, 1);
    mbar_init(&drain_bar[0], 1);
    mbar_init(&drain_bar[1], 1);
    mbar_init(&dp_free[0], 1);
    mbar_init(&dp_free[1], 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == W_MMA) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  int n_items = 0;
  {
    KvWalk<SPARSE> w;
    for (w.init(); w.next(p, qpos0);) ++n_items;
  }

  if (n_items > 0) {
    if (warp == W_TMA) {
      if (lane == 0) {
        tma_prefetch_desc(&tmK);
        tma_prefetch_desc(&tmV);
        mbar_expect_tx(qdo_full, 2 * TILE_BYTES);
        tma_load_4d(sQ, &tmQ, qdo_full, 0, hq, t * BT, b);
        tma_load_4d(sQ + HALF_BYTES, &tmQ, qdo_full, 64, hq, t * BT, b);
        tma_load_4d(sdO, &tmdO, qdo_full, 0, hq, t * BT, b);
        tma_load_4d(sdO + HALF_BYTES, &tmdO, qdo_full, 64, hq, t * BT, b);
        uint32_t n = 0;
        bool ok = true;
        KvWalk<SPARSE> w;
        for (w.init(); w.next(p, qpos0);) {
          const int j = w.j;
          const int ks = n % K_STAGES, vs = n % V_STAGES;
          if (!mbar_wait(&k_empty[ks], ((n / K_STAGES) & 1) ^ 1, abort_flag)) { ok = false; break; }
          mbar_expect_tx(&k_full[ks], TILE_BYTES);
          tma_load_4d(sK + ks * TILE_BYTES, &tmK, &k_full[ks], 0, hk, j * BT, b);
          tma_load_4d(sK + ks * TILE_BYTES + HALF_BYTES, &tmK, &k_full[ks], 64, hk, j * BT, b);
          if (!mbar_wait(&v_empty[vs], ((n / V_STAGES) & 1) ^ 1, abort_flag)) { ok = false; break; }
          mbar_expect_tx(&v_full[vs], TILE_BYTES);
          tma_load_4d(sV + vs * TILE_BYTES, &tmV, &v_full[vs], 0, hk, j * BT, b);
          tma_load_4d(sV + vs * TILE_BYTES + HALF_BYTES, &tmV, &v_full[vs], 64, hk, j * BT, b);
          ++n;
        }
        if (!ok) {
          report(p.status, ZX_ERR_TIMEOUT, /*site=*/21, (int)n);
          const uint64_t t0 = globaltimer_ns();
          while (globaltimer_ns() - t0 < 2000000ull) {
          }
        }
      }
    } else if (warp == W_MMA) {
      // MMA warp of the "early" products: S(n+1) = Q K(n+1)^T as soon as the compute warps hold S(n) in
      // registers, dP(n+1) = dO V(n+1)^T into the dP buffer that dQ(n-1) has released. A tcgen05.mma leaves
      // its issuing thread only when the tensor core has room for it, so these must not queue behind dQ(n)
      // in one warp's instruction stream: dQ has a warp of its own (below). dP lives in two TMEM buffers
      // used alternately; with that the compute warps never wait for a tensor result of their own item.
      constexpr uint32_t idesc_kk = make_idesc(BT, BT, 1, 1, 0, 0);
      const uint32_t t_s = tmem_base, t_dp = tmem_base + 128;
      const uint64_t q_addr = base_kmajor(smem_u32(sQ)), do_addr = base_kmajor(smem_u32(sdO));
      const uint64_t k_k0 = base_kmajor(smem_u32(sK)), v_k0 = base_kmajor(smem_u32(sV));
      bool ok = mbar_wait_w(qdo_full, 0, abort_flag);
      ok = ok && mbar_wait_w(&k_full[0], 0, abort_flag);
      ok = ok && mbar_wait_w(&v_full[0], 0, abort_flag);
      tc_fence_after();
      if (ok) {
        umma_ss_k8_kmajor_w<HALF_BYTES / 16>(t_s, q_addr, k_k0, idesc_kk, 0u);
        umma_commit_w(s_full);
        umma_ss_k8_kmajor_w<HALF_BYTES / 16>(t_dp, do_addr, v_k0, idesc_kk, 0u);
        umma_commit_w(dp_full);
        umma_commit_w(&v_empty[0]);
      }
      int n = 0;
      for (; n + 1 < n_items && ok; ++n) {
        const int ksn = (n + 1) % K_STAGES, vsn = (n + 1) % V_STAGES;
        const uint64_t kn_addr = desc_advance(k_k0, (uint32_t)ksn * TILE_BYTES);
        const uint64_t vn_addr = desc_advance(v_k0, (uint32_t)vsn * TILE_BYTES);
        if (!mbar_wait_w(s_read, n & 1, abort_flag)) { ok = false; break; }
        if (!mbar_wait_w(&k_full[ksn], ((n + 1) / K_STAGES) & 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        umma_ss_k8_kmajor_w<HALF_BYTES / 16>(t_s, q_addr, kn_addr, idesc_kk, 0u);
        umma_commit_w(s_full);
        // buffer (n+1) & 1 held dS(n-1), which dQ(n-1) reads
        if (n >= 1 && !mbar_wait_w(&dp_free[(n + 1) & 1], ((n - 1) >> 1) & 1, abort_flag)) { ok = false; break; }
        if (!mbar_wait_w(&v_full[vsn], ((n + 1) / V_STAGES) & 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        umma_ss_k8_kmajor_w<HALF_BYTES / 16>(t_dp + (uint32_t)((n + 1) & 1) * 256, do_addr, vn_addr, idesc_kk, 0u);
        umma_commit_w(dp_full);
        umma_commit_w(&v_empty[vsn]);   // V(n+1) is only read by dP(n+1)
      }
      if (!ok) {
        if (lane == 0) report(p.status, ZX_ERR_TIMEOUT, /*site=*/22, n);
        umma_commit_w(&drain_bar[0]);
        const uint64_t t0 = globaltimer_ns();
        while (!mbar_try_wait(&drain_bar[0], 0) && globaltimer_ns() - t0 < 50000000ull) {
        }
      }
    } else if (warp == W_MMA_DQ) {
      // MMA warp of dQ(n) += dS(n) K(n): A = dS from the dP buffer of item n, B = K(n) read transposed
      constexpr uint32_t idesc_tm = make_idesc(BT, HD, 1, 1, 0, 1);
      const uint32_t t_dp = tmem_base + 128, t_dq = tmem_base + 256;
      const uint64_t k_mn0 = base_mnmajor(smem_u32(sK));
      bool ok = true;
      int n = 0;
      for (; n < n_items && ok; ++n) {
        const int ks = n % K_STAGES;
        if (!mbar_wait_w(ds_ready, n & 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        if (lane == 0) ZX_TRACE(n, 8);
        umma_ts_k8_w<8, 16, 24, 64, 72, 80, 88>(t_dq, t_dp + (uint32_t)(n & 1) * 256,
                                                 desc_advance(k_mn0, (uint32_t)ks * TILE_BYTES), idesc_tm, n > 0 ? 1u : 0u);
        umma_commit_w(&k_empty[ks]);        // K(n) has now served S(n) and dQ(n)
        umma_commit_w(&dp_free[n & 1]);
        if (lane == 0) ZX_TRACE(n, 9);
      }
      if (ok) umma_commit_w(acc_done);
      if (!ok) {
        if (lane == 0) report(p.status, ZX_ERR_TIMEOUT, /*site=*/22, n);
        umma_commit_w(&drain_bar[1]);
        const uint64_t t0 = globaltimer_ns();
        while (!mbar_try_wait(&drain_bar[1], 0) && globaltimer_ns() - t0 < 50000000ull) {
        }
      }
    } else {
      // Two warpgroups: warpgroup wg owns key columns [64 wg, 64 wg + 64) of every query row.
      const int wg = warp >> 2;
      const int lq = warp & 3;
      const int r = lq * 32 + lane;  // query row == TMEM lane
      const int col0 = wg * 64;
      const uint32_t lane_base = (uint32_t)(lq * 32) << 16;
      const uint32_t t_s = tmem_base + lane_base + col0, t_dp0 = tmem_base + lane_base + 128 + col0;
      const size_t stat_idx = ((size_t)b * p.Hq + hq) * p.Sq + (size_t)t * BT + r;
      const float lse2 = p.lse[stat_idx] * LOG2E;
      const float dlt = p.delta[stat_idx];
      const int my_qpos = qpos0 + r;
      uint32_t n = 0;
      bool ok = true;
      KvWalk<SPARSE> walk;
      for (walk.init(); walk.next(p, qpos0);) {
        const int kpos0 = walk.kpos0;
        if (!wait_warp(s_full, n & 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        if (threadIdx.x == 0) ZX_TRACE(n, 0);
        if (threadIdx.x == 160) ZX_TRACE(n, 11);
        uint32_t sr[64];
        tmem_ld_32x32b_x32(t_s + 0, sr);
        tmem_ld_32x32b_x32(t_s + 32, sr + 32);
        tmem_wait_ld();
        if (threadIdx.x == 0) ZX_TRACE(n, 1);
        tc_fence_before();
        mbar_arrive_warp(s_read);
        const bool diag = p.causal && (kpos0 + BT - 1 > qpos0);
        const int kp = kpos0 + col0;
        const float2 sl2 = make_float2(p.scale_log2, p.scale_log2);
        const float2 nl2 = make_float2(-lse2, -lse2);
        static_for<32>([&](auto idx) {   // packed fp32x2 math: two key columns per instruction
          constexpr int c = decltype(idx)::value;
          const float2 x = __ffma2_rn(make_float2(__uint_as_float(sr[2 * c]), __uint_as_float(sr[2 * c + 1])), sl2, nl2);
          const float2 e = exp2_pair<c, DQ_POLY_EVERY>(x);
          sr[2 * c] = __float_as_uint(e.x);
          sr[2 * c + 1] = __float_as_uint(e.y);
        });
        if (diag) {   // only tiles on the diagonal pay for the per-element mask
#pragma unroll
          for (int c = 0; c < 64; ++c)
            if (kp + c > my_qpos) sr[c] = 0u;
        }
        if (threadIdx.x == 0) ZX_TRACE(n, 2);
        if (threadIdx.x == 160) ZX_TRACE(n, 12);
        if (!wait_warp(dp_full, n & 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        if (threadIdx.x == 0) ZX_TRACE(n, 3);
        const uint32_t t_dp = t_dp0 + (n & 1) * 256;   // the two dP buffers sit at columns 128 and 384
        uint32_t dp[64];
        tmem_ld_32x32b_x32(t_dp + 0, dp);
        tmem_ld_32x32b_x32(t_dp + 32, dp + 32);
        tmem_wait_ld();
        if (threadIdx.x == 0) ZX_TRACE(n, 4);
        {
          uint32_t dsp[32];
          const float2 ndl = make_float2(-dlt, -dlt);
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            const float2 t2 = __fadd2_rn(make_float2(__uint_as_float(dp[2 * e]), __uint_as_float(dp[2 * e + 1])), ndl);
            const float2 d = __fmul2_rn(make_float2(__uint_as_float(sr[2 * e]), __uint_as_float(sr[2 * e + 1])), t2);
            dsp[e] = pack_bf16x2(d.x, d.y);
          }
          if (threadIdx.x == 0) ZX_TRACE(n, 6);
          tmem_st_32x32b_x32(t_dp, dsp);   // bf16 dS for this half, over the columns this thread just read
        }
        tmem_wait_st();
        if (threadIdx.x == 0) ZX_TRACE(n, 5);
        if (threadIdx.x == 160) ZX_TRACE(n, 13);
        tc_fence_before();
        mbar_arrive_warp(ds_ready);
        ++n;
      }
      if (ok) ok = wait_warp(acc_done, 0, abort_flag);
      tc_fence_after();
      if (ok && ZX_IN_BOUNDS(p.status, t * BT + r, p.Sq, 25)) {
        float* dq_row = p.dq + (((size_t)b * p.Sq + (size_t)t * BT + r) * p.Hq + hq) * HD + col0;
#pragma unroll
        for (int ci = 0; ci < 2; ++ci) {
          uint32_t a[32];
          tmem_ld_32x32b_x32(tmem_base + lane_base + 256 + col0 + ci * 32, a);
          tmem_wait_ld();
          float4* dst = reinterpret_cast<float4*>(dq_row + ci * 32);
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            float4 v = make_float4(__uint_as_float(a[4 * e]) * p.scale, __uint_as_float(a[4 * e + 1]) * p.scale,
                                   __uint_as_float(a[4 * e + 2]) * p.scale, __uint_as_float(a[4 * e + 3]) * p.scale);
            if (p.dq_accumulate) {
              const float4 o = dst[e];
              v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
            }
            dst[e] = v;
          }
        }
      }
      if (!ok && lane == 0) report(p.status, ZX_ERR_TIMEOUT, /*site=*/23, (int)n);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == W_MMA) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

CUtensorMap make_qkv_map(const void* base, int B, int S, int H, int64_t tok_stride) {
  uint64_t dims[4] = {(uint64_t)HD, (uint64_t)H, (uint64_t)S, (uint64_t)B};
  uint64_t strides[3] = {(uint64_t)HD * 2, (uint64_t)tok_stride * 2, (uint64_t)S * (uint64_t)tok_stride * 2};
  uint32_t box[4] = {64, 1, 128, 1};
  return make_tma_map(base, 2, 4, dims, strides, box, TmaSwizzle::B128);
}

template <typename K>
void set_smem(K kern, int bytes, const char* name) {
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e != cudaSuccess)
    throw std::runtime_error(std::string(name) + ": cannot raise shared memory limit: " + cudaGetErrorString(e));
}

}  // namespace

void launch_attn_bwd(const AttnBwdArgs& a) {
  check_attn_common(a.Hq, a.Hkv, a.Sq, a.Skv, a.q_layout, a.kv_layout);
  if (a.Sq == 0 || a.Skv == 0 || a.B == 0) return;
  if (a.compute_delta) {
    const size_t rows = (size_t)a.B * a.Sq * a.Hq;
    const int wpb = 8;
    attn_delta_kernel<<<(unsigned)((rows + wpb - 1) / wpb), wpb * 32, 0, a.stream>>>(
        (const __nv_bfloat16*)a.o, (const __nv_bfloat16*)a.d_o, a.delta, a.B, a.Sq, a.Hq);
  }
  CUtensorMap tmQ = make_qkv_map(a.q, a.B, a.Sq, a.Hq, a.q_tok_stride);
  CUtensorMap tmdO = make_qkv_map(a.d_o, a.B, a.Sq, a.Hq, (int64_t)a.Hq * HD);
  CUtensorMap tmK = make_qkv_map(a.k, a.B, a.Skv, a.Hkv, a.k_tok_stride);
  CUtensorMap tmV = make_qkv_map(a.v, a.B, a.Skv, a.Hkv, a.v_tok_stride);
  BwdParams p;
  p.B = a.B; p.Hq = a.Hq; p.Hkv = a.Hkv; p.Sq = a.Sq; p.Skv = a.Skv;
  p.scale = a.scale;
  p.scale_log2 = a.scale * LOG2E;
  p.causal = a.mask.causal; p.window_blocks = a.mask.window_blocks; p.global_every = a.mask.global_every;
  p.n_q_tiles = a.Sq / BT;
  p.n_kv_tiles = a.Skv / BT;
  p.q_tiles_per_chunk = a.q_layout.chunk_len / BT;
  p.kv_tiles_per_chunk = a.kv_layout.chunk_len / BT;
  for (int c = 0; c < kAttnMaxChunks; ++c) {
    p.q_chunk_pos[c] = c < a.q_layout.n_chunks ? a.q_layout.chunk_pos[c] : 0;
    p.kv_chunk_pos[c] = c < a.kv_layout.n_chunks ? a.kv_layout.chunk_pos[c] : 0;
  }
  p.lse = a.lse; p.delta = a.delta;
  p.dq = a.dq; p.dk = a.dk; p.dv = a.dv;
  p.dq_accumulate = a.dq_accumulate;
  if (a.pull_bytes % 16 != 0) throw std::runtime_error("attn_bwd: pull size must be a multiple of 16 bytes");
  p.pull_src = (const uint4*)a.pull_src;
  p.pull_dst = (uint4*)a.pull_dst;
  p.pull_nvec = a.pull_src != nullptr ? a.pull_bytes / 16 : 0;
  p.trace = a.trace;
  p.status = a.status;
  static PerDeviceOnce once;
  bool& configured = once.current();
  if (!configured) {
    set_smem(attn_bwd_dkdv_kernel<false>, DKDV_SMEM, "attn_bwd_dkdv");
    set_smem(attn_bwd_dkdv_kernel<true>, DKDV_SMEM, "attn_bwd_dkdv (windowed)");
    set_smem(attn_bwd_dq_kernel<false>, DQ_SMEM, "attn_bwd_dq");
    set_smem(attn_bwd_dq_kernel<true>, DQ_SMEM, "attn_bwd_dq (windowed)");
    configured = true;
  }
  const unsigned grid_kv = p.n_kv_tiles * a.B * a.Hkv, grid_q = p.n_q_tiles * a.B * a.Hq;
  if (p.window_blocks > 0) {
    attn_bwd_dkdv_kernel<true><<<grid_kv, DKDV_THREADS, DKDV_SMEM, a.stream>>>(tmQ, tmdO, tmK, tmV, p);
    attn_bwd_dq_kernel<true><<<grid_q, NUM_THREADS, DQ_SMEM, a.stream>>>(tmQ, tmdO, tmK, tmV, p);
  } else {
    attn_bwd_dkdv_kernel<false><<<grid_kv, DKDV_THREADS, DKDV_SMEM, a.stream>>>(tmQ, tmdO, tmK, tmV, p);
    attn_bwd_dq_kernel<false><<<grid_q, NUM_THREADS, DQ_SMEM, a.stream>>>(tmQ, tmdO, tmK, tmV, p);
  }
}

}  // namespace zx
