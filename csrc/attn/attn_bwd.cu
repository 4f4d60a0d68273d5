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
#include "../common/tma_host.h"
#include "attn.h"

namespace zx {

void check_attn_common(int Hq, int Hkv, int Sq, int Skv, const AttnLayout& ql, const AttnLayout& kl);

namespace {

constexpr int HD = 128;
constexpr int BT = 128;                    // tile edge in tokens (both Q and KV)
constexpr int TILE_BYTES = BT * HD * 2;    // 32 KB
constexpr int HALF_BYTES = TILE_BYTES / 2; // one 64-wide d chunk
constexpr int NUM_THREADS = 320;           // 8 compute warps (two warpgroups) + TMA warp + MMA warp
constexpr int DKDV_THREADS = 352;          // ... + peer-pull warp
constexpr int W_TMA = 8, W_MMA = 9, W_PULL = 10;
constexpr int N_COMPUTE = 256;             // compute threads
constexpr int TMEM_COLS = 512;
constexpr float LOG2E = 1.4426950408889634f;

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

// clock stamp of one pipeline event (dQ kernel, first CTA only, when a trace buffer is given)
#define ZX_TRACE(iter, slot)                                                          \
  do {                                                                                \
    if (p.trace != nullptr && blockIdx.x == 0 && (iter) < 64) p.trace[(iter) * 16 + (slot)] = clock64(); \
  } while (0)

__device__ __forceinline__ bool tile_allowed(const BwdParams& p, int qpos0, int kpos0) {
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
__device__ __forceinline__ int q_tile_pos(const BwdParams& p, int t) {
  return p.q_chunk_pos[t / p.q_tiles_per_chunk] + (t % p.q_tiles_per_chunk) * BT;
}
__device__ __forceinline__ int kv_tile_pos(const BwdParams& p, int j) {
  return p.kv_chunk_pos[j / p.kv_tiles_per_chunk] + (j % p.kv_tiles_per_chunk) * BT;
}
__device__ __forceinline__ bool wait_warp(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  const bool ok = mbar_wait(bar, parity, abort_flag);
  return __all_sync(0xffffffffu, ok);
}
__device__ __forceinline__ void bulk_load_1d(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(smem_dst)),
               "l"(reinterpret_cast<uint64_t>(gsrc)), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
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
// ... and their k-step variants: one add each. K-major: 16 elements of d; MN-major: 16 token rows.
__device__ __forceinline__ uint64_t desc_kmajor(uint64_t base, int k) {
  return desc_advance(base, (k >> 2) * HALF_BYTES + (k & 3) * 32);
}
__device__ __forceinline__ uint64_t desc_mnmajor(uint64_t base, int k) { return desc_advance(base, k * 16 * 128); }

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
constexpr int DKDV_SMEM = 2 * TILE_BYTES /*K,V*/ + 4 * TILE_BYTES /*Q,dO x2*/ + 3 * 2 * BT * 4 /*lse,delta,lse2*/ +
                          1024 + 256;

__global__ void __launch_bounds__(DKDV_THREADS, 1)
attn_bwd_dkdv_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmdO,
                     const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV, BwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;
  uint8_t* sV = smem + TILE_BYTES;
  uint8_t* sQ = smem + 2 * TILE_BYTES;   // [2]
  uint8_t* sdO = smem + 4 * TILE_BYTES;  // [2]
  float* s_lse = reinterpret_cast<float*>(smem + 6 * TILE_BYTES);  // [2][128] written by TMA
  float* s_delta = s_lse + 2 * BT;                                 // [2][128] written by TMA
  float* s_lse2 = s_delta + 2 * BT;                                // [2][128] written by compute warps
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_lse2 + 2 * BT);
  uint64_t* kv_full = bars;         // 1
  uint64_t* qdo_full = bars + 1;    // [2]
  uint64_t* qdo_empty = bars + 3;   // [2]
  uint64_t* s_full = bars + 5;      // 1
  uint64_t* dp_full = bars + 6;     // 1
  uint64_t* p_ready = bars + 7;     // 1 (128 arrivals)
  uint64_t* ds_ready = bars + 8;    // 1 (128 arrivals)
  uint64_t* acc_done = bars + 9;    // 1
  uint64_t* drain_bar = bars + 10;  // 1
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 11);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  int bid = blockIdx.x;
  const int hk = bid % p.Hkv;
  bid /= p.Hkv;
  const int b = bid % p.B;
  const int j = bid / p.B;  // KV tile; early tiles (most work under a causal mask) run first
  const int G = p.Hq / p.Hkv;
  const int kpos0 = kv_tile_pos(p, j);

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&qdo_full[s], 1);
      mbar_init(&qdo_empty[s], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(dp_full, 1);
    mbar_init(p_ready, N_COMPUTE);
    mbar_init(ds_ready, N_COMPUTE);
    mbar_init(acc_done, 1);
    mbar_init(drain_bar, 1);
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

  // number of (head, q tile) items this CTA processes: identical in every role
  int n_items = 0;
  for (int t = 0; t < p.n_q_tiles; ++t)
    if (tile_allowed(p, q_tile_pos(p, t), kpos0)) ++n_items;
  n_items *= G;

  if (warp == W_PULL) warp_pull_slice(p.pull_src, p.pull_dst, p.pull_nvec, lane);

  if (n_items > 0 && warp < W_PULL) {
    if (warp == W_TMA) {
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
          for (int t = 0; t < p.n_q_tiles; ++t) {
            if (!tile_allowed(p, q_tile_pos(p, t), kpos0)) continue;
            const int s = n & 1;
            if (!mbar_wait(&qdo_empty[s], ((n >> 1) & 1) ^ 1, abort_flag)) { ok = false; break; }
            mbar_expect_tx(&qdo_full[s], 2 * TILE_BYTES + 2 * BT * 4);
            tma_load_4d(sQ + s * TILE_BYTES, &tmQ, &qdo_full[s], 0, hq, t * BT, b);
            tma_load_4d(sQ + s * TILE_BYTES + HALF_BYTES, &tmQ, &qdo_full[s], 64, hq, t * BT, b);
            tma_load_4d(sdO + s * TILE_BYTES, &tmdO, &qdo_full[s], 0, hq, t * BT, b);
            tma_load_4d(sdO + s * TILE_BYTES + HALF_BYTES, &tmdO, &qdo_full[s], 64, hq, t * BT, b);
            const size_t row0 = ((size_t)b * p.Hq + hq) * p.Sq + (size_t)t * BT;
            bulk_load_1d(s_lse + s * BT, p.lse + row0, BT * 4, &qdo_full[s]);
            bulk_load_1d(s_delta + s * BT, p.delta + row0, BT * 4, &qdo_full[s]);
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
    } else if (warp == W_MMA) {
      // ------------------------------- MMA issuer ---------------------------------
      {  // all 32 lanes run this loop; the instructions themselves are issued by one elected lane
        constexpr uint32_t idesc_kk = make_idesc(BT, BT, 1, 1, 0, 0);  // both operands K-major
        constexpr uint32_t idesc_tm = make_idesc(BT, HD, 1, 1, 0, 1);  // A from TMEM, B MN-major
        const uint32_t t_s = tmem_base, t_dp = tmem_base + 128, t_dv = tmem_base + 256, t_dk = tmem_base + 384;
        const uint64_t k_addr = base_kmajor(smem_u32(sK)), v_addr = base_kmajor(smem_u32(sV));
        const uint64_t q_k0 = base_kmajor(smem_u32(sQ)), do_k0 = base_kmajor(smem_u32(sdO));
        const uint64_t q_mn0 = base_mnmajor(smem_u32(sQ)), do_mn0 = base_mnmajor(smem_u32(sdO));
        bool ok = mbar_wait_w(kv_full, 0, abort_flag);
        ok = ok && mbar_wait_w(&qdo_full[0], 0, abort_flag);
        tc_fence_after();
        if (ok) {
#pragma unroll
          for (int k = 0; k < 8; ++k) umma_ss_w(t_s, desc_kmajor(k_addr, k), desc_kmajor(q_k0, k), idesc_kk, k > 0);
          umma_commit_w(s_full);
#pragma unroll
          for (int k = 0; k < 8; ++k) umma_ss_w(t_dp, desc_kmajor(v_addr, k), desc_kmajor(do_k0, k), idesc_kk, k > 0);
          umma_commit_w(dp_full);
        }
        int n = 0;
        for (; n < n_items && ok; ++n) {
          const int s = n & 1, sn = (n + 1) & 1;
          const bool has_next = n + 1 < n_items;
          const uint64_t q_addr = desc_advance(q_mn0, (uint32_t)s * TILE_BYTES);     // read transposed
          const uint64_t do_addr = desc_advance(do_mn0, (uint32_t)s * TILE_BYTES);   // read transposed
          const uint64_t qn_addr = desc_advance(q_k0, (uint32_t)sn * TILE_BYTES);
          const uint64_t don_addr = desc_advance(do_k0, (uint32_t)sn * TILE_BYTES);
          // dV += P^T dO
          if (!mbar_wait_w(p_ready, n & 1, abort_flag)) { ok = false; break; }
          tc_fence_after();
#pragma unroll
          for (int k = 0; k < 8; ++k) umma_ts_w(t_dv, t_s + (k >> 2) * 64 + (k & 3) * 8, desc_mnmajor(do_addr, k), idesc_tm, (n > 0 || k > 0));
          if (has_next) {
            if (!mbar_wait_w(&qdo_full[sn], ((n + 1) >> 1) & 1, abort_flag)) { ok = false; break; }
            tc_fence_after();
#pragma unroll
            for (int k = 0; k < 8; ++k) umma_ss_w(t_s, desc_kmajor(k_addr, k), desc_kmajor(qn_addr, k), idesc_kk, k > 0);
            umma_commit_w(s_full);
          }
          // dK += dS^T Q
          if (!mbar_wait_w(ds_ready, n & 1, abort_flag)) { ok = false; break; }
          tc_fence_after();
#pragma unroll
          for (int k = 0; k < 8; ++k) umma_ts_w(t_dk, t_dp + (k >> 2) * 64 + (k & 3) * 8, desc_mnmajor(q_addr, k), idesc_tm, (n > 0 || k > 0));
          umma_commit_w(&qdo_empty[s]);
          if (has_next) {
#pragma unroll
            for (int k = 0; k < 8; ++k)
              umma_ss_w(t_dp, desc_kmajor(v_addr, k), desc_kmajor(don_addr, k), idesc_kk, k > 0);
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
      // Two warpgroups: warpgroup wg owns query columns [64 wg, 64 wg + 64) of every KV row.
      const int wg = warp >> 2;
      const int lq = warp & 3;                 // TMEM lane quarter
      const int r = lq * 32 + lane;            // KV row of this thread == TMEM lane
      const int col0 = wg * 64;
      const uint32_t lane_base = (uint32_t)(lq * 32) << 16;
      const uint32_t t_s = tmem_base + lane_base + col0, t_dp = tmem_base + lane_base + 128 + col0;
      const int my_kpos = kpos0 + r;
      uint32_t n = 0;
      bool ok = true;
      for (int g = 0; g < G && ok; ++g) {
        for (int t = 0; t < p.n_q_tiles; ++t) {
          const int qpos0 = q_tile_pos(p, t);
          if (!tile_allowed(p, qpos0, kpos0)) continue;
          const int s = n & 1;
          if (!wait_warp(&qdo_full[s], (n >> 1) & 1, abort_flag)) { ok = false; break; }
          if (!wait_warp(s_full, n & 1, abort_flag)) { ok = false; break; }
          tc_fence_after();
          uint32_t sr[64];
          tmem_ld_32x32b_x32(t_s + 0, sr);
          tmem_ld_32x32b_x32(t_s + 32, sr + 32);
          tmem_wait_ld();
          const bool diag = p.causal && (kpos0 + BT - 1 > qpos0);
          // packed fp32x2 math: two query columns per instruction
          const float2* lse_nat2 = reinterpret_cast<const float2*>(s_lse + s * BT + col0);
          const int qp = qpos0 + col0;   // column c is query qp + c; it sees this key iff my_kpos <= qp + c
          const float2 sl2 = make_float2(p.scale_log2, p.scale_log2);
          const float2 nlog2e = make_float2(-LOG2E, -LOG2E);
#pragma unroll
          for (int c = 0; c < 32; ++c) {
            const float2 x = __ffma2_rn(make_float2(__uint_as_float(sr[2 * c]), __uint_as_float(sr[2 * c + 1])), sl2,
                                        __fmul2_rn(lse_nat2[c], nlog2e));
            float p0 = fast_exp2(x.x), p1 = fast_exp2(x.y);
            if (diag) {
              if (my_kpos > qp + 2 * c) p0 = 0.f;
              if (my_kpos > qp + 2 * c + 1) p1 = 0.f;
            }
            sr[2 * c] = __float_as_uint(p0);
            sr[2 * c + 1] = __float_as_uint(p1);
          }
          {
            // bf16 P^T for this half goes over the first 32 columns of the half this thread just read
            uint32_t pk[32];
#pragma unroll
            for (int c = 0; c < 32; ++c) pk[c] = pack_bf16x2(__uint_as_float(sr[2 * c]), __uint_as_float(sr[2 * c + 1]));
            tmem_st_32x32b_x32(t_s, pk);
          }
          tmem_wait_st();
          tc_fence_before();
          mbar_arrive(p_ready);
          if (!wait_warp(dp_full, n & 1, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const float2* dl2 = reinterpret_cast<const float2*>(s_delta + s * BT + col0);
          uint32_t dp[64];
          tmem_ld_32x32b_x32(t_dp + 0, dp);
          tmem_ld_32x32b_x32(t_dp + 32, dp + 32);
          tmem_wait_ld();
          {
            uint32_t dsp[32];
#pragma unroll
            for (int e = 0; e < 32; ++e) {
              const float2 dl = dl2[e];
              const float2 t2 = __fadd2_rn(make_float2(__uint_as_float(dp[2 * e]), __uint_as_float(dp[2 * e + 1])),
                                           make_float2(-dl.x, -dl.y));
              const float2 d = __fmul2_rn(make_float2(__uint_as_float(sr[2 * e]), __uint_as_float(sr[2 * e + 1])), t2);
              dsp[e] = pack_bf16x2(d.x, d.y);
            }
            tmem_st_32x32b_x32(t_dp, dsp);
          }
          tmem_wait_st();
          tc_fence_before();
          mbar_arrive(ds_ready);
          ++n;
        }
      }
      // epilogue: add dV and scale * dK into the (possibly remote) fp32 accumulators; each
      // warpgroup drains its 64 columns of both accumulators
      if (ok) ok = wait_warp(acc_done, 0, abort_flag);
      tc_fence_after();
      if (ok) {
        const size_t row_off = (((size_t)b * p.Skv + (size_t)j * BT + r) * p.Hkv + hk) * HD + col0;
        float* dv_row = p.dv + row_off;
        float* dk_row = p.dk + row_off;
#pragma unroll
        for (int ci = 0; ci < 2; ++ci) {
          uint32_t a[32];
          tmem_ld_32x32b_x32(tmem_base + lane_base + 256 + col0 + ci * 32, a);
          tmem_wait_ld();
#pragma unroll
          for (int e = 0; e < 8; ++e)
            red_add_v4_sys(dv_row + ci * 32 + e * 4, __uint_as_float(a[4 * e]), __uint_as_float(a[4 * e + 1]),
                           __uint_as_float(a[4 * e + 2]), __uint_as_float(a[4 * e + 3]));
        }
#pragma unroll
        for (int ci = 0; ci < 2; ++ci) {
          uint32_t a[32];
          tmem_ld_32x32b_x32(tmem_base + lane_base + 384 + col0 + ci * 32, a);
          tmem_wait_ld();
#pragma unroll
          for (int e = 0; e < 8; ++e)
            red_add_v4_sys(dk_row + ci * 32 + e * 4, __uint_as_float(a[4 * e]) * p.scale,
                           __uint_as_float(a[4 * e + 1]) * p.scale, __uint_as_float(a[4 * e + 2]) * p.scale,
                           __uint_as_float(a[4 * e + 3]) * p.scale);
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

// ------------------------------------------------------------------------------------------
// dQ
// ------------------------------------------------------------------------------------------
constexpr int DQ_SMEM = 2 * TILE_BYTES /*Q,dO*/ + 4 * TILE_BYTES /*K,V x2*/ + 1024 + 256;

__global__ void __launch_bounds__(NUM_THREADS, 1)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmdO,
                   const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV, BwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sdO = smem + TILE_BYTES;
  uint8_t* sK = smem + 2 * TILE_BYTES;  // [2]
  uint8_t* sV = smem + 4 * TILE_BYTES;  // [2]
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 6 * TILE_BYTES);
  uint64_t* qdo_full = bars;       // 1
  uint64_t* kv_full = bars + 1;    // [2]
  uint64_t* kv_empty = bars + 3;   // [2]
  uint64_t* s_full = bars + 5;     // 1
  uint64_t* dp_full = bars + 6;    // 1
  uint64_t* s_read = bars + 7;     // 1 (128 arrivals)
  uint64_t* ds_ready = bars + 8;   // 1 (128 arrivals)
  uint64_t* acc_done = bars + 9;   // 1
  uint64_t* drain_bar = bars + 10; // 1
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 11);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  int bid = blockIdx.x;
  const int hq = bid % p.Hq;
  bid /= p.Hq;
  const int b = bid % p.B;
  const int t = p.n_q_tiles - 1 - bid / p.B;  // late Q tiles (most work) first
  const int hk = hq / (p.Hq / p.Hkv);
  const int qpos0 = q_tile_pos(p, t);

  if (threadIdx.x == 0) {
    mbar_init(qdo_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(dp_full, 1);
    mbar_init(s_read, N_COMPUTE);
    mbar_init(ds_ready, N_COMPUTE);
    mbar_init(acc_done, 1);
    mbar_init(drain_bar, 1);
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
  for (int j = 0; j < p.n_kv_tiles; ++j)
    if (tile_allowed(p, qpos0, kv_tile_pos(p, j))) ++n_items;

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
        for (int j = 0; j < p.n_kv_tiles; ++j) {
          if (!tile_allowed(p, qpos0, kv_tile_pos(p, j))) continue;
          const int s = n & 1;
          if (!mbar_wait(&kv_empty[s], ((n >> 1) & 1) ^ 1, abort_flag)) { ok = false; break; }
          mbar_expect_tx(&kv_full[s], 2 * TILE_BYTES);
          tma_load_4d(sK + s * TILE_BYTES, &tmK, &kv_full[s], 0, hk, j * BT, b);
          tma_load_4d(sK + s * TILE_BYTES + HALF_BYTES, &tmK, &kv_full[s], 64, hk, j * BT, b);
          tma_load_4d(sV + s * TILE_BYTES, &tmV, &kv_full[s], 0, hk, j * BT, b);
          tma_load_4d(sV + s * TILE_BYTES + HALF_BYTES, &tmV, &kv_full[s], 64, hk, j * BT, b);
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
      {  // all 32 lanes run this loop; the instructions themselves are issued by one elected lane
        constexpr uint32_t idesc_kk = make_idesc(BT, BT, 1, 1, 0, 0);
        constexpr uint32_t idesc_tm = make_idesc(BT, HD, 1, 1, 0, 1);
        const uint32_t t_s = tmem_base, t_dp = tmem_base + 128, t_dq = tmem_base + 256;
        const uint64_t q_addr = base_kmajor(smem_u32(sQ)), do_addr = base_kmajor(smem_u32(sdO));
        const uint64_t k_k0 = base_kmajor(smem_u32(sK)), v_k0 = base_kmajor(smem_u32(sV));
        const uint64_t k_mn0 = base_mnmajor(smem_u32(sK));
        bool ok = mbar_wait_w(qdo_full, 0, abort_flag);
        ok = ok && mbar_wait_w(&kv_full[0], 0, abort_flag);
        tc_fence_after();
        if (ok) {
#pragma unroll
          for (int k = 0; k < 8; ++k) umma_ss_w(t_s, desc_kmajor(q_addr, k), desc_kmajor(k_k0, k), idesc_kk, k > 0);
          umma_commit_w(s_full);
#pragma unroll
          for (int k = 0; k < 8; ++k) umma_ss_w(t_dp, desc_kmajor(do_addr, k), desc_kmajor(v_k0, k), idesc_kk, k > 0);
          umma_commit_w(dp_full);
        }
        int n = 0;
        for (; n < n_items && ok; ++n) {
          const int s = n & 1, sn = (n + 1) & 1;
          const bool has_next = n + 1 < n_items;
          const uint64_t k_addr = desc_advance(k_mn0, (uint32_t)s * TILE_BYTES);   // read transposed
          const uint64_t kn_addr = desc_advance(k_k0, (uint32_t)sn * TILE_BYTES);
          const uint64_t vn_addr = desc_advance(v_k0, (uint32_t)sn * TILE_BYTES);
          if (has_next) {
            if (!mbar_wait_w(s_read, n & 1, abort_flag)) { ok = false; break; }
            if (!mbar_wait_w(&kv_full[sn], ((n + 1) >> 1) & 1, abort_flag)) { ok = false; break; }
            tc_fence_after();
#pragma unroll
            for (int k = 0; k < 8; ++k) umma_ss_w(t_s, desc_kmajor(q_addr, k), desc_kmajor(kn_addr, k), idesc_kk, k > 0);
            umma_commit_w(s_full);
          }
          if (!mbar_wait_w(ds_ready, n & 1, abort_flag)) { ok = false; break; }
          tc_fence_after();
          if (lane == 0) ZX_TRACE(n, 8);
#pragma unroll
          for (int k = 0; k < 8; ++k) umma_ts_w(t_dq, t_dp + (k >> 2) * 64 + (k & 3) * 8, desc_mnmajor(k_addr, k), idesc_tm, (n > 0 || k > 0));
          umma_commit_w(&kv_empty[s]);
          if (lane == 0) ZX_TRACE(n, 9);
          if (has_next) {
#pragma unroll
            for (int k = 0; k < 8; ++k)
              umma_ss_w(t_dp, desc_kmajor(do_addr, k), desc_kmajor(vn_addr, k), idesc_kk, k > 0);
            umma_commit_w(dp_full);
          }
          if (lane == 0) ZX_TRACE(n, 10);
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
      // Two warpgroups: warpgroup wg owns key columns [64 wg, 64 wg + 64) of every query row.
      const int wg = warp >> 2;
      const int lq = warp & 3;
      const int r = lq * 32 + lane;  // query row == TMEM lane
      const int col0 = wg * 64;
      const uint32_t lane_base = (uint32_t)(lq * 32) << 16;
      const uint32_t t_s = tmem_base + lane_base + col0, t_dp = tmem_base + lane_base + 128 + col0;
      const size_t stat_idx = ((size_t)b * p.Hq + hq) * p.Sq + (size_t)t * BT + r;
      const float lse2 = p.lse[stat_idx] * LOG2E;
      const float dlt = p.delta[stat_idx];
      const int my_qpos = qpos0 + r;
      uint32_t n = 0;
      bool ok = true;
      for (int j = 0; j < p.n_kv_tiles; ++j) {
        const int kpos0 = kv_tile_pos(p, j);
        if (!tile_allowed(p, qpos0, kpos0)) continue;
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
        mbar_arrive(s_read);
        const bool diag = p.causal && (kpos0 + BT - 1 > qpos0);
        const int kp = kpos0 + col0;
        const float2 sl2 = make_float2(p.scale_log2, p.scale_log2);
        const float2 nl2 = make_float2(-lse2, -lse2);
#pragma unroll
        for (int c = 0; c < 32; ++c) {   // packed fp32x2 math: two key columns per instruction
          const float2 x = __ffma2_rn(make_float2(__uint_as_float(sr[2 * c]), __uint_as_float(sr[2 * c + 1])), sl2, nl2);
          float p0 = fast_exp2(x.x), p1 = fast_exp2(x.y);
          if (diag) {
            if (kp + 2 * c > my_qpos) p0 = 0.f;
            if (kp + 2 * c + 1 > my_qpos) p1 = 0.f;
          }
          sr[2 * c] = __float_as_uint(p0);
          sr[2 * c + 1] = __float_as_uint(p1);
        }
        if (threadIdx.x == 0) ZX_TRACE(n, 2);
        if (threadIdx.x == 160) ZX_TRACE(n, 12);
        if (!wait_warp(dp_full, n & 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        if (threadIdx.x == 0) ZX_TRACE(n, 3);
        uint32_t dp[64];
        tmem_ld_32x32b_x32(t_dp + 0, dp);
        tmem_ld_32x32b_x32(t_dp + 32, dp + 32);
        tmem_wait_ld();
        if (threadIdx.x == 0) ZX_TRACE(n, 4);
        {
          uint32_t dsp[32];
#pragma unroll
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
        mbar_arrive(ds_ready);
        ++n;
      }
      if (ok) ok = wait_warp(acc_done, 0, abort_flag);
      tc_fence_after();
      if (ok) {
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
  static bool configured = false;
  if (!configured) {
    set_smem(attn_bwd_dkdv_kernel, DKDV_SMEM, "attn_bwd_dkdv");
    set_smem(attn_bwd_dq_kernel, DQ_SMEM, "attn_bwd_dq");
    configured = true;
  }
  attn_bwd_dkdv_kernel<<<p.n_kv_tiles * a.B * a.Hkv, DKDV_THREADS, DKDV_SMEM, a.stream>>>(tmQ, tmdO, tmK, tmV, p);
  attn_bwd_dq_kernel<<<p.n_q_tiles * a.B * a.Hq, NUM_THREADS, DQ_SMEM, a.stream>>>(tmQ, tmdO, tmK, tmV, p);
}

}  // namespace zx
