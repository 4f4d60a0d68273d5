// Flash-attention forward for sm_100a (head_dim 128, bf16 in, fp32 softmax/accumulate).
//
// One CTA owns two adjacent 128-row Q tiles of one head and walks the KV buffer once:
//   warp 8      TMA producer: Q once, then K/V tiles through a 2-stage ring (plain per-CTA loads)
//   warp 9      MMA issuer:   S_i = Q_i K^T  (SS form) and O_i += P_i V (A = P read from TMEM)
//   warp 10     optional peer pull: copies this CTA's slice of the next ring step's K/V from the
//               owning GPU into local staging with plain P2P loads while the tiles compute
//   warps 0-3   softmax of Q tile 0, one thread per row, S/P/O live in TMEM
//   warps 4-7   softmax of Q tile 1
// The two softmax groups ping-pong so the tensor core always has the other tile's MMAs to run.
// TMEM (512 columns): S0 | S1 | O0 | O1, with the bf16 P_i written over the first half of S_i.
// O is only rescaled when a row's running max grew by more than 2^8 (the final 1/l makes the
// result exact either way). Causal / block-sparse masks come from global token positions, so the
// same kernel serves plain sequences, zigzag context-parallel shards and every ring step; with
// merge_prev it folds its result into the O/LSE left by the previous ring step.
#include "../common/ptx.cuh"
#include "../common/tma_host.h"
#include "attn.h"

namespace zx {

namespace {

constexpr int HD = 128;
constexpr int BQ = 128;
constexpr int BKV = 128;
constexpr int TILE_BYTES = BQ * HD * 2;   // 32 KB
constexpr int HALF_BYTES = TILE_BYTES / 2; // one 64-wide d chunk: 128 rows x 128 B
constexpr int KV_STAGES = 2;
constexpr int NUM_THREADS = 352;  // 8 softmax warps + TMA + MMA + peer-pull warp
constexpr int TMEM_COLS = 512;
constexpr int SMEM_BYTES = 2 * TILE_BYTES + KV_STAGES * 2 * TILE_BYTES + 1024 + 256;
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

__device__ __forceinline__ bool tile_allowed(const FwdParams& p, int qpos0, int kpos0) {
  if (p.causal && kpos0 > qpos0) return false;  // tiles are 128-aligned in position space
  if (p.window_blocks > 0) {
    const int qb = qpos0 >> 7, kb = kpos0 >> 7;
    const int dist = qb >= kb ? qb - kb : kb - qb;
    const bool in_window = dist < p.window_blocks;
    const bool is_global = p.global_every > 0 && (kb % p.global_every) == 0;
    if (!in_window && !is_global) return false;
  }
  return true;
}
__device__ __forceinline__ int q_tile_pos(const FwdParams& p, int t) {
  return p.q_chunk_pos[t / p.q_tiles_per_chunk] + (t % p.q_tiles_per_chunk) * BQ;
}
__device__ __forceinline__ int kv_tile_pos(const FwdParams& p, int j) {
  return p.kv_chunk_pos[j / p.kv_tiles_per_chunk] + (j % p.kv_tiles_per_chunk) * BKV;
}

// warp-uniform bounded wait
__device__ __forceinline__ bool wait_warp(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  const bool ok = mbar_wait(bar, parity, abort_flag);
  return __all_sync(0xffffffffu, ok);
}

__global__ void __launch_bounds__(NUM_THREADS, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, FwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;                                   // [2][32 KB]
  uint8_t* sK = smem + 2 * TILE_BYTES;                  // [KV_STAGES][32 KB]
  uint8_t* sV = sK + KV_STAGES * TILE_BYTES;            // [KV_STAGES][32 KB]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sV + KV_STAGES * TILE_BYTES);
  uint64_t* q_full = bars;          // 1
  uint64_t* k_full = bars + 1;      // [2]
  uint64_t* v_full = bars + 3;      // [2]
  uint64_t* k_empty = bars + 5;     // [2]
  uint64_t* v_empty = bars + 7;     // [2]
  uint64_t* s_full = bars + 9;      // [2]
  uint64_t* p_ready = bars + 11;    // [2]
  uint64_t* o_done = bars + 13;     // [2]
  uint64_t* drain_bar = bars + 15;  // 1
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // block -> (q pair, head, batch); the heaviest (latest) q tiles are scheduled first
  const int n_pairs = (p.n_q_tiles + 1) >> 1;
  int bid = blockIdx.x;
  const int h = bid % p.Hq;
  bid /= p.Hq;
  const int b = bid % p.B;
  const int pair = n_pairs - 1 - bid / p.B;
  const int hkv = h / (p.Hq / p.Hkv);
  const int qt0 = pair * 2;
  const bool has_q1 = qt0 + 1 < p.n_q_tiles;
  const int qpos[2] = {q_tile_pos(p, qt0), has_q1 ? q_tile_pos(p, qt0 + 1) : 0};

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < KV_STAGES; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&k_empty[s], 1);
      mbar_init(&v_empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&p_ready[i], 4);   // one arrival per softmax warp
      mbar_init(&o_done[i], 1);
    }
    mbar_init(drain_bar, 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 9) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 8) {
    // ------------------------------- TMA producer -------------------------------
    if (lane == 0) {
      tma_prefetch_desc(&tmQ);
      tma_prefetch_desc(&tmK);
      tma_prefetch_desc(&tmV);
      mbar_expect_tx(q_full, has_q1 ? 2 * TILE_BYTES : TILE_BYTES);
      for (int i = 0; i < (has_q1 ? 2 : 1); ++i) {
        tma_load_4d(sQ + i * TILE_BYTES, &tmQ, q_full, 0, h, (qt0 + i) * BQ, b);
        tma_load_4d(sQ + i * TILE_BYTES + HALF_BYTES, &tmQ, q_full, 64, h, (qt0 + i) * BQ, b);
      }
      uint32_t n = 0;
      bool ok = true;
      for (int j = 0; j < p.n_kv_tiles; ++j) {
        const int kpos0 = kv_tile_pos(p, j);
        const bool need = tile_allowed(p, qpos[0], kpos0) || (has_q1 && tile_allowed(p, qpos[1], kpos0));
        if (!need) continue;
        const int s = n % KV_STAGES;
        const uint32_t ph = (n / KV_STAGES) & 1;
        if (!mbar_wait(&k_empty[s], ph ^ 1, abort_flag)) { ok = false; break; }
        mbar_expect_tx(&k_full[s], TILE_BYTES);
        tma_load_4d(sK + s * TILE_BYTES, &tmK, &k_full[s], 0, hkv, j * BKV, b);
        tma_load_4d(sK + s * TILE_BYTES + HALF_BYTES, &tmK, &k_full[s], 64, hkv, j * BKV, b);
        if (!mbar_wait(&v_empty[s], ph ^ 1, abort_flag)) { ok = false; break; }
        mbar_expect_tx(&v_full[s], TILE_BYTES);
        tma_load_4d(sV + s * TILE_BYTES, &tmV, &v_full[s], 0, hkv, j * BKV, b);
        tma_load_4d(sV + s * TILE_BYTES + HALF_BYTES, &tmV, &v_full[s], 64, hkv, j * BKV, b);
        ++n;
      }
      if (!ok) {
        report(p.status, ZX_ERR_TIMEOUT, /*site=*/11, (int)n);
        // give loads already in flight a bounded moment to land before the CTA retires
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 2000000ull) {
        }
      }
    }
  } else if (warp == 9) {
    // ------------------------------- MMA issuer ---------------------------------
    {  // all 32 lanes run this loop; the instructions themselves are issued by one elected lane
      constexpr uint32_t idesc_qk = make_idesc(BQ, BKV, 1, 1, 0, 0);
      constexpr uint32_t idesc_pv = make_idesc(BQ, HD, 1, 1, 0, 1);
      // Base descriptors are built once; every MMA below only adds a constant to them.
      const uint64_t q_desc0 = make_smem_desc_sw128(smem_u32(sQ), 16, 1024);          // K-major tiles
      const uint64_t k_desc0 = make_smem_desc_sw128(smem_u32(sK), 16, 1024);
      const uint64_t v_desc0 = make_smem_desc_sw128(smem_u32(sV), HALF_BYTES, 1024);  // read transposed (MN-major)
      bool ok = mbar_wait_w(q_full, 0, abort_flag);
      tc_fence_after();
      uint32_t n = 0;
      int pend_stage[2] = {-1, -1};
      uint32_t pend_phase[2] = {0, 0};
      uint32_t cnt[2] = {0, 0};
      int prev_stage = -1;

      auto issue_pv = [&](int i) -> bool {
        if (!mbar_wait_w(&p_ready[i], (cnt[i] - 1) & 1, abort_flag)) return false;
        if (!mbar_wait_w(&v_full[pend_stage[i]], pend_phase[i], abort_flag)) return false;
        tc_fence_after();
        const uint64_t v_desc = desc_advance(v_desc0, (uint32_t)pend_stage[i] * TILE_BYTES);
        const uint32_t o_tmem = tmem_base + 256 + i * 128;
        const uint32_t p_tmem = tmem_base + i * 128;
#pragma unroll
        for (int k = 0; k < BKV / 16; ++k) {
          umma_ts_w(o_tmem, p_tmem + k * 8, desc_advance(v_desc, k * 16 * 128), idesc_pv,
                  (cnt[i] > 1 || k > 0) ? 1u : 0u);
        }
        umma_commit_w(&o_done[i]);
        pend_stage[i] = -1;
        return true;
      };

      for (int j = 0; j < p.n_kv_tiles && ok; ++j) {
        const int kpos0 = kv_tile_pos(p, j);
        const bool need[2] = {tile_allowed(p, qpos[0], kpos0), has_q1 && tile_allowed(p, qpos[1], kpos0)};
        if (!need[0] && !need[1]) continue;
        const int s = n % KV_STAGES;
        const uint32_t ph = (n / KV_STAGES) & 1;
        bool k_waited = false;
        for (int i = 0; i < 2 && ok; ++i) {
          if (pend_stage[i] >= 0) {
            if (!issue_pv(i)) { ok = false; break; }
          }
          if (!need[i]) continue;
          if (!k_waited) {
            if (!mbar_wait_w(&k_full[s], ph, abort_flag)) { ok = false; break; }
            tc_fence_after();
            k_waited = true;
          }
          const uint64_t q_desc = desc_advance(q_desc0, (uint32_t)i * TILE_BYTES);
          const uint64_t k_desc = desc_advance(k_desc0, (uint32_t)s * TILE_BYTES);
#pragma unroll
          for (int k = 0; k < HD / 16; ++k) {
            const uint32_t off = (k >> 2) * HALF_BYTES + (k & 3) * 32;
            umma_ss_w(tmem_base + i * 128, desc_advance(q_desc, off), desc_advance(k_desc, off), idesc_qk,
                    k > 0 ? 1u : 0u);
          }
          umma_commit_w(&s_full[i]);
          pend_stage[i] = s;
          pend_phase[i] = ph;
          ++cnt[i];
        }
        if (!ok) break;
        umma_commit_w(&k_empty[s]);
        if (prev_stage >= 0) umma_commit_w(&v_empty[prev_stage]);
        prev_stage = s;
        ++n;
      }
      for (int i = 0; i < 2 && ok; ++i) {
        if (pend_stage[i] >= 0) {
          if (!issue_pv(i)) ok = false;
        }
      }
      if (!ok) {
        if (lane == 0) report(p.status, ZX_ERR_TIMEOUT, /*site=*/12, (int)n);
        umma_commit_w(drain_bar);
        const uint64_t t0 = globaltimer_ns();
        while (!mbar_try_wait(drain_bar, 0) && globaltimer_ns() - t0 < 50000000ull) {
        }
      }
    }
  } else if (warp == 10) {
    // ------------------------------- peer pull ----------------------------------
    warp_pull_slice(p.pull_src, p.pull_dst, p.pull_nvec, lane);
  } else {
    // ------------------------------- softmax groups -----------------------------
    const int i = warp >> 2;       // which Q tile
    const int q = warp & 3;        // TMEM lane quarter
    const int r = q * 32 + lane;   // row within the tile
    const bool active = (i == 0) || has_q1;
    if (active) {
      const uint32_t lane_base = (uint32_t)(q * 32) << 16;
      const uint32_t s_tmem = tmem_base + lane_base + i * 128;
      const uint32_t o_tmem = tmem_base + lane_base + 256 + i * 128;
      const int my_qpos = qpos[i] + r;
      float m_used = NEG_BIG, l = 0.f;
      uint32_t cnt = 0;
      bool ok = true;
      for (int j = 0; j < p.n_kv_tiles; ++j) {
        const int kpos0 = kv_tile_pos(p, j);
        if (!tile_allowed(p, qpos[i], kpos0)) continue;
        if (!wait_warp(&s_full[i], cnt & 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        uint32_t sr[128];
        tmem_ld_32x32b_x32(s_tmem + 0, sr);
        tmem_ld_32x32b_x32(s_tmem + 32, sr + 32);
        tmem_ld_32x32b_x32(s_tmem + 64, sr + 64);
        tmem_ld_32x32b_x32(s_tmem + 96, sr + 96);
        tmem_wait_ld();
        const bool diag = p.causal && (kpos0 + BKV - 1 > qpos[i]);
        // four independent running maxima / sums instead of one dependent chain of 128 operations
        float mx4[4] = {NEG_BIG, NEG_BIG, NEG_BIG, NEG_BIG};
        if (diag) {
#pragma unroll
          for (int c = 0; c < 128; ++c) {
            float v = __uint_as_float(sr[c]);
            v = (kpos0 + c > my_qpos) ? NEG_BIG : v;
            sr[c] = __float_as_uint(v);
            mx4[c & 3] = fmaxf(mx4[c & 3], v);
          }
        } else {
#pragma unroll
          for (int c = 0; c < 128; ++c) mx4[c & 3] = fmaxf(mx4[c & 3], __uint_as_float(sr[c]));
        }
        const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
        const float m_cur = mx * p.scale_log2;
        if (cnt == 0) {
          m_used = m_cur;
        } else {
          const bool grow = m_cur > m_used + RESCALE_THRESHOLD;
          if (__any_sync(0xffffffffu, grow)) {
            const float alpha = grow ? fast_exp2(m_used - m_cur) : 1.f;
            if (grow) {
              m_used = m_cur;
              l *= alpha;
            }
            if (!wait_warp(&o_done[i], (cnt - 1) & 1, abort_flag)) { ok = false; break; }
            tc_fence_after();
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              uint32_t orow[32];
              tmem_ld_32x32b_x32(o_tmem + c * 32, orow);
              tmem_wait_ld();
#pragma unroll
              for (int e = 0; e < 32; ++e) orow[e] = __float_as_uint(__uint_as_float(orow[e]) * alpha);
              tmem_st_32x32b_x32(o_tmem + c * 32, orow);
            }
          }
        }
        uint32_t pk[64];
        // The row sum runs as two packed fp32x2 accumulators (two independent chains of 32 adds),
        // the scale-and-shift as packed FMAs, and every fourth pair of exponentials on the FMA pipe.
        float2 sum_a = make_float2(0.f, 0.f), sum_b = make_float2(0.f, 0.f);
        const float2 sl2 = make_float2(p.scale_log2, p.scale_log2);
        const float2 nm2 = make_float2(-m_used, -m_used);
        auto softmax_pair = [&](auto idx) {
          constexpr int c = decltype(idx)::value;
          const float2 x = __ffma2_rn(make_float2(__uint_as_float(sr[2 * c]), __uint_as_float(sr[2 * c + 1])), sl2, nm2);
          const float2 pe = exp2_pair<c>(x);
          if (c & 1) sum_b = __fadd2_rn(sum_b, pe);
          else sum_a = __fadd2_rn(sum_a, pe);
          pk[c] = pack_bf16x2(pe.x, pe.y);
        };
        static_for<64>(softmax_pair);
        l += (sum_a.x + sum_a.y) + (sum_b.x + sum_b.y);
        tmem_st_32x32b_x32(s_tmem + 0, pk);
        tmem_st_32x32b_x32(s_tmem + 32, pk + 32);
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive_warp(&p_ready[i]);
        ++cnt;
      }

      // ------------------------------- epilogue -----------------------------------
      const int row_tok = (qt0 + i) * BQ + r;
      __nv_bfloat16* orow_g = p.O + (((size_t)b * p.Sq + row_tok) * p.Hq + h) * HD;
      float* lse_g = p.LSE + ((size_t)b * p.Hq + h) * p.Sq + row_tok;
      if (ok && cnt > 0) {
        ok = wait_warp(&o_done[i], (cnt - 1) & 1, abort_flag);
        tc_fence_after();
      }
      if (ok && cnt > 0) {
        const float inv_l = l > 0.f ? 1.f / l : 0.f;
        const float lse_cur = l > 0.f ? (m_used + __log2f(l)) * 0.6931471805599453f : -INFINITY;
        float w_prev = 0.f, w_cur = inv_l, lse_new = lse_cur;
        if (p.merge_prev) {
          const float lse_prev = *lse_g;
          const float mxl = fmaxf(lse_prev, lse_cur);
          if (mxl == -INFINITY) {
            w_prev = 0.f; w_cur = 0.f; lse_new = -INFINITY;
          } else {
            const float e_prev = __expf(lse_prev - mxl), e_cur = __expf(lse_cur - mxl);
            lse_new = mxl + __logf(e_prev + e_cur);
            w_prev = e_prev / (e_prev + e_cur);
            w_cur = e_cur / (e_prev + e_cur) * inv_l;
          }
        }
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t orow[32];
          tmem_ld_32x32b_x32(o_tmem + c * 32, orow);
          tmem_wait_ld();
          uint4* dst = reinterpret_cast<uint4*>(orow_g + c * 32);
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            float f[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(orow[g * 8 + e]) * w_cur;
            if (p.merge_prev) {
              const uint4 pv = dst[g];
              const float2 a = unpack_bf16x2(pv.x), bb = unpack_bf16x2(pv.y), cc = unpack_bf16x2(pv.z),
                           dd = unpack_bf16x2(pv.w);
              f[0] += w_prev * a.x; f[1] += w_prev * a.y; f[2] += w_prev * bb.x; f[3] += w_prev * bb.y;
              f[4] += w_prev * cc.x; f[5] += w_prev * cc.y; f[6] += w_prev * dd.x; f[7] += w_prev * dd.y;
            }
            uint4 o4;
            o4.x = pack_bf16x2(f[0], f[1]);
            o4.y = pack_bf16x2(f[2], f[3]);
            o4.z = pack_bf16x2(f[4], f[5]);
            o4.w = pack_bf16x2(f[6], f[7]);
            dst[g] = o4;
          }
        }
        *lse_g = lse_new;
      } else if (ok && cnt == 0 && !p.merge_prev) {
        // nothing visible to this tile in this call: an empty softmax
        uint4* dst = reinterpret_cast<uint4*>(orow_g);
#pragma unroll
        for (int g = 0; g < 16; ++g) dst[g] = make_uint4(0, 0, 0, 0);
        *lse_g = -INFINITY;
      }
      if (!ok && lane == 0) report(p.status, ZX_ERR_TIMEOUT, /*site=*/13, (int)cnt);
    }
  }

  // ------------------------------- teardown -------------------------------------
  tc_fence_before();
  __syncthreads();
  if (warp == 9) {
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

}  // namespace

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
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess)
      throw std::runtime_error(std::string("attn_fwd: cannot raise shared memory limit: ") + cudaGetErrorString(e));
    configured = true;
  }
  const int n_pairs = (p.n_q_tiles + 1) / 2;
  const int grid = n_pairs * a.Hq * a.B;
  attn_fwd_kernel<<<grid, NUM_THREADS, SMEM_BYTES, a.stream>>>(tmQ, tmK, tmV, p);
}

}  // namespace zx
