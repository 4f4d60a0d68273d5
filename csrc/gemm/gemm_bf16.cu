// Persistent bf16 GEMM for sm_100a: C[M,N] = A[M,K] * B[N,K]^T (+ D), fp32 accumulation in TMEM.
//
//  * operands are staged by TMA (128-byte swizzle, per-CTA loads) through a 4-deep mbarrier ring,
//  * one elected thread issues tcgen05.mma 128x256x16 into one of two 256-column TMEM accumulators,
//  * four epilogue warps drain the other accumulator with tcgen05.ld while the next tile computes.
//
// Either operand may be "MN-major" (stored transposed, i.e. [K, M] / [K, N] row-major), which is
// what dgrad (dX = dY * W) and wgrad (dW = dY^T * X) need, so no transposes are ever materialised.
// Every wait is bounded; on a timeout the kernel records a Status and unwinds through the normal
// teardown (outstanding copies drained, TMEM freed).
#include "../common/ptx.cuh"
#include "../common/device_once.h"
#include "../common/tma_host.h"
#include "gemm.h"

namespace zx {

namespace {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int STAGES = 4;
constexpr int UMMA_K = 16;
constexpr int A_STAGE_BYTES = BM * BK * 2;  // 16 KB
constexpr int B_STAGE_BYTES = BN * BK * 2;  // 32 KB
constexpr int CHUNK_BYTES = 64 * BK * 2;    // one 64-wide MN chunk of an MN-major tile: 8 KB
constexpr int NUM_THREADS = 224;   // TMA, MMA, four epilogue warps, one peer-pull warp
constexpr int W_PULL = 6;
constexpr int TMEM_COLS = 512;
// Output staging for the TMA-store epilogue: per epilogue warp two slabs of 32 rows x 64 bf16 columns (128-byte
// rows, 128-byte swizzle), written from registers and handed to cp.async.bulk.tensor stores.
constexpr int SLAB_BYTES = 32 * 128;
constexpr int STAGING_BYTES = 4 * 2 * SLAB_BYTES;   // 32 KB
constexpr int SMEM_BYTES = STAGES * (A_STAGE_BYTES + B_STAGE_BYTES) + STAGING_BYTES + 1024 /*align*/ + 256 /*barriers*/;
static_assert(SMEM_BYTES <= 227 * 1024, "gemm shared memory");

struct KParams {
  int M, N, K;
  int ldc, ldd;
  void* C;
  const void* D;
  int out_fp32;
  int d_mode;  // 0: none, 1: bf16 addend, 2: fp32 addend
  int tma_store;  // plain bf16 output: the epilogue goes through shared memory and TMA stores
  int num_m, num_n;
  const uint4* pull_src;
  uint4* pull_dst;
  size_t pull_nvec;
  int scatter_ranks, scatter_rows_per_rank, scatter_src_rank;
  __nv_bfloat16* scatter_base[8];
  Status* status;
};

__device__ __forceinline__ void tile_coords(int t, int num_m, int num_n, int& tm, int& tn) {
  constexpr int GM = 16;
  const int per_group = GM * num_n;
  const int g = t / per_group;
  const int first_m = g * GM;
  const int gsize = min(num_m - first_m, GM);
  const int r = t - g * per_group;
  tm = first_m + r % gsize;
  tn = r / gsize;
}

template <bool A_MN, bool B_MN>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmC, const __grid_constant__ CUtensorMap tmD, KParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * A_STAGE_BYTES;
  uint8_t* sStage = smem + STAGES * (A_STAGE_BYTES + B_STAGE_BYTES);   // 1024-byte aligned: STAGES * 48 KB above smem
  uint64_t* bars = reinterpret_cast<uint64_t*>(sStage + STAGING_BYTES);
  uint64_t* full = bars;                 // [STAGES]
  uint64_t* empty = bars + STAGES;       // [STAGES]
  uint64_t* acc_full = bars + 2 * STAGES;      // [2]
  uint64_t* acc_empty = bars + 2 * STAGES + 2; // [2]
  uint64_t* drain_bar = bars + 2 * STAGES + 4; // [1]
  uint64_t* d_full = bars + 2 * STAGES + 5;    // [4] addend slab of epilogue warp q has landed
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 9);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_tiles = p.num_m * p.num_n;
  const int num_kb = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 4);   // one arrival per epilogue warp
    }
    mbar_init(drain_bar, 1);
    for (int w = 0; w < 4; ++w) mbar_init(&d_full[w], 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------- TMA producer -------------------------------
    if (lane == 0) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      uint32_t it = 0;  // global k-block counter -> stage / phase
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int tm, tn;
        tile_coords(t, p.num_m, p.num_n, tm, tn);
        const int m0 = tm * BM, n0 = tn * BN;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&empty[s], ph ^ 1, abort_flag)) { ok = false; break; }
          mbar_expect_tx(&full[s], A_STAGE_BYTES + B_STAGE_BYTES);
          uint8_t* a_dst = sA + s * A_STAGE_BYTES;
          uint8_t* b_dst = sB + s * B_STAGE_BYTES;
          if (!A_MN) {
            tma_load_2d(a_dst, &tmA, &full[s], kb * BK, m0);
          } else {
#pragma unroll
            for (int c = 0; c < BM / 64; ++c) tma_load_2d(a_dst + c * CHUNK_BYTES, &tmA, &full[s], m0 + c * 64, kb * BK);
          }
          if (!B_MN) {
            tma_load_2d(b_dst, &tmB, &full[s], kb * BK, n0);
          } else {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c) tma_load_2d(b_dst + c * CHUNK_BYTES, &tmB, &full[s], n0 + c * 64, kb * BK);
          }
        }
      }
      if (!ok) {
        report(p.status, ZX_ERR_TIMEOUT, /*site=*/1, (int)it);
        // Loads already issued still land in shared memory: give them a bounded moment to finish.
        const uint32_t outstanding = it < (uint32_t)STAGES ? it : (uint32_t)STAGES;
        for (uint32_t j = 0; j < outstanding; ++j) {
          const uint32_t jt = it - 1 - j;
          uint64_t t0 = globaltimer_ns();
          while (!mbar_try_wait(&full[jt % STAGES], (jt / STAGES) & 1) && globaltimer_ns() - t0 < 50000000ull) {
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer ---------------------------------
    {  // all 32 lanes run this loop; the instructions themselves are issued by one elected lane
      constexpr uint32_t idesc = make_idesc(BM, BN, 1, 1, A_MN ? 1 : 0, B_MN ? 1 : 0);
      // stage-0 descriptors; stages and k-steps are reached by adding constants
      const uint64_t a_desc0 = A_MN ? make_smem_desc_sw128(smem_u32(sA), CHUNK_BYTES, 1024)
                                    : make_smem_desc_sw128(smem_u32(sA), 16, 1024);
      const uint64_t b_desc0 = B_MN ? make_smem_desc_sw128(smem_u32(sB), CHUNK_BYTES, 1024)
                                    : make_smem_desc_sw128(smem_u32(sB), 16, 1024);
      uint32_t it = 0;
      uint32_t lt = 0;  // local tile counter
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++lt) {
        const uint32_t buf = lt & 1;
        if (!mbar_wait_w(&acc_empty[buf], ((lt >> 1) & 1) ^ 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * BN;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % STAGES;
          if (!mbar_wait_w(&full[s], (it / STAGES) & 1, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint64_t a_base = desc_advance(a_desc0, (uint32_t)s * A_STAGE_BYTES);
          const uint64_t b_base = desc_advance(b_desc0, (uint32_t)s * B_STAGE_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t a_desc = desc_advance(a_base, A_MN ? k * UMMA_K * 128 : k * UMMA_K * 2);
            const uint64_t b_desc = desc_advance(b_base, B_MN ? k * UMMA_K * 128 : k * UMMA_K * 2);
            umma_ss_w(d_tmem, a_desc, b_desc, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit_w(&empty[s]);  // stage is free once these MMAs have read it
        }
        if (ok) umma_commit_w(&acc_full[buf]);
      }
      if (!ok) {
        if (lane == 0) report(p.status, ZX_ERR_TIMEOUT, /*site=*/2, (int)it);
        umma_commit_w(drain_bar);
        uint64_t t0 = globaltimer_ns();
        while (!mbar_try_wait(drain_bar, 0) && globaltimer_ns() - t0 < 50000000ull) {
        }
      }
    }
  } else if (warp == W_PULL) {
    // ------------------------------- peer pull ----------------------------------
    warp_pull_slice<16>(p.pull_src, p.pull_dst, p.pull_nvec, lane);
  } else {
    // ------------------------------- epilogue warps -----------------------------
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    uint32_t lt = 0;
    uint32_t d_phase = 0;    // parity of this warp's addend barrier
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++lt) {
      int tm, tn;
      tile_coords(t, p.num_m, p.num_n, tm, tn);
      const uint32_t buf = lt & 1;
      if (!mbar_wait(&acc_full[buf], (lt >> 1) & 1, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const int row = tm * BM + q * 32 + lane;
      const bool row_ok = row < p.M;
      if (p.tma_store) {
        // Thread-per-row stores put 16 bytes of 32 different rows into every store instruction, and the L2 traffic
        // of those partial sectors cost the main loop 4-17 % of its throughput. Here each 64-column chunk of the
        // warp's 32 rows is packed to bf16, written to a swizzled slab in shared memory (chunk c of row r at
        // position c ^ (r % 8): conflict-free per quarter warp) and stored by the TMA unit as whole 128-byte
        // lines; the unit also clips rows and columns beyond the matrix.
        // A bf16 addend takes the same road in the other direction: its slab is loaded by the TMA unit into the
        // staging slab (rows and columns beyond the matrix read as zero) while the accumulator is unpacked.
        uint8_t* slabs = sStage + q * 2 * SLAB_BYTES;
        if (tm * BM + q * 32 < p.M) {
#pragma unroll 1
          for (int cc = 0; cc < BN / 64; ++cc) {
            const int col0 = tn * BN + cc * 64;
            if (col0 >= p.N) break;
            uint8_t* slab = slabs + (cc & 1) * SLAB_BYTES;
            if (lane == 0) {
              tma_store_wait_read<1>();   // the store that read this slab two chunks ago is done with it
              if (p.d_mode == 1) {
                mbar_expect_tx(&d_full[q], SLAB_BYTES);
                tma_load_2d(slab, &tmD, &d_full[q], col0, tm * BM + q * 32);
              }
            }
            __syncwarp();   // lane 0 has seen the slab free
            uint8_t* srow = slab + lane * 128;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              uint32_t r[32];
              tmem_ld_32x32b_x32(tmem_addr(tmem_base, q * 32, buf * BN + cc * 64 + h * 32), r);
              tmem_wait_ld();
              if (p.d_mode == 1) {
                if (h == 0) {
                  if (!mbar_wait(&d_full[q], d_phase, abort_flag)) { ok = false; break; }
                  d_phase ^= 1u;
                }
#pragma unroll
                for (int c4 = 0; c4 < 4; ++c4) {   // fp32 accumulator + addend, rounded to bf16 once
                  uint4* cell = reinterpret_cast<uint4*>(srow + (((h * 4 + c4) ^ (lane & 7)) << 4));
                  const uint4 d = *cell;
                  const float2 a0 = unpack_bf16x2(d.x), a1 = unpack_bf16x2(d.y), a2 = unpack_bf16x2(d.z),
                               a3 = unpack_bf16x2(d.w);
                  const uint32_t* f = r + 8 * c4;
                  *cell = make_uint4(pack_bf16x2(__uint_as_float(f[0]) + a0.x, __uint_as_float(f[1]) + a0.y),
                                     pack_bf16x2(__uint_as_float(f[2]) + a1.x, __uint_as_float(f[3]) + a1.y),
                                     pack_bf16x2(__uint_as_float(f[4]) + a2.x, __uint_as_float(f[5]) + a2.y),
                                     pack_bf16x2(__uint_as_float(f[6]) + a3.x, __uint_as_float(f[7]) + a3.y));
                }
              } else {
#pragma unroll
                for (int c4 = 0; c4 < 4; ++c4) {
                  const uint32_t* f = r + 8 * c4;
                  *reinterpret_cast<uint4*>(srow + (((h * 4 + c4) ^ (lane & 7)) << 4)) =
                      make_uint4(pack_bf16x2(__uint_as_float(f[0]), __uint_as_float(f[1])),
                                 pack_bf16x2(__uint_as_float(f[2]), __uint_as_float(f[3])),
                                 pack_bf16x2(__uint_as_float(f[4]), __uint_as_float(f[5])),
                                 pack_bf16x2(__uint_as_float(f[6]), __uint_as_float(f[7])));
                }
              }
            }
            if (!ok) break;
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              tma_store_2d(&tmC, slab, col0, tm * BM + q * 32);
              tma_store_commit();
            }
          }
        }
        if (!ok) break;
        tc_fence_before();
        mbar_arrive_warp(&acc_empty[buf]);
        continue;
      }
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(tmem_addr(tmem_base, q * 32, buf * BN + c * 32), r);
        tmem_wait_ld();
        const int col0 = tn * BN + c * 32;
        if (row_ok && col0 < p.N) {
          // N is a multiple of 8, so validity is decided per group of 8 columns.
          if (p.d_mode == 1) {
            const uint4* dsrc = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(p.D) +
                                                               (size_t)row * p.ldd + col0);
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              if (col0 + g * 8 < p.N) {
                uint4 v = dsrc[g];
                const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  float2 f = unpack_bf16x2(w[j]);
                  r[g * 8 + 2 * j] = __float_as_uint(__uint_as_float(r[g * 8 + 2 * j]) + f.x);
                  r[g * 8 + 2 * j + 1] = __float_as_uint(__uint_as_float(r[g * 8 + 2 * j + 1]) + f.y);
                }
              }
            }
          } else if (p.d_mode == 2) {
            const float4* dsrc =
                reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.D) + (size_t)row * p.ldd + col0);
#pragma unroll
            for (int g = 0; g < 8; ++g) {
              if (col0 + g * 4 < p.N) {
                float4 v = dsrc[g];
                r[g * 4 + 0] = __float_as_uint(__uint_as_float(r[g * 4 + 0]) + v.x);
                r[g * 4 + 1] = __float_as_uint(__uint_as_float(r[g * 4 + 1]) + v.y);
                r[g * 4 + 2] = __float_as_uint(__uint_as_float(r[g * 4 + 2]) + v.z);
                r[g * 4 + 3] = __float_as_uint(__uint_as_float(r[g * 4 + 3]) + v.w);
              }
            }
          }
          if (p.out_fp32) {
            float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(p.C) + (size_t)row * p.ldc + col0);
#pragma unroll
            for (int g = 0; g < 8; ++g) {
              if (col0 + g * 4 < p.N)
                dst[g] = make_float4(__uint_as_float(r[g * 4]), __uint_as_float(r[g * 4 + 1]),
                                     __uint_as_float(r[g * 4 + 2]), __uint_as_float(r[g * 4 + 3]));
            }
          } else {
            __nv_bfloat16* crow = reinterpret_cast<__nv_bfloat16*>(p.C) + (size_t)row * p.ldc;
            if (p.scatter_ranks > 0) {
              // reduce-scatter fused into the epilogue: this partial row goes to the slot its owner keeps for us
              const int owner = row / p.scatter_rows_per_rank;
              if (!ZX_IN_BOUNDS(p.status, owner, p.scatter_ranks, 4)) continue;
              crow = p.scatter_base[owner] +
                     ((size_t)p.scatter_src_rank * p.scatter_rows_per_rank + (row - owner * p.scatter_rows_per_rank)) * p.ldc;
            }
            uint4* dst = reinterpret_cast<uint4*>(crow + col0);
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              if (col0 + g * 8 < p.N) {
                uint4 v;
                v.x = pack_bf16x2(__uint_as_float(r[g * 8 + 0]), __uint_as_float(r[g * 8 + 1]));
                v.y = pack_bf16x2(__uint_as_float(r[g * 8 + 2]), __uint_as_float(r[g * 8 + 3]));
                v.z = pack_bf16x2(__uint_as_float(r[g * 8 + 4]), __uint_as_float(r[g * 8 + 5]));
                v.w = pack_bf16x2(__uint_as_float(r[g * 8 + 6]), __uint_as_float(r[g * 8 + 7]));
                dst[g] = v;
              }
            }
          }
        }
      }
      tc_fence_before();
      mbar_arrive_warp(&acc_empty[buf]);
    }
    if (!ok && lane == 0) report(p.status, ZX_ERR_TIMEOUT, /*site=*/3, (int)lt);
    if (p.tma_store && lane == 0) tma_store_wait<0>();   // shared memory must outlive the stores that read it
  }

  // ------------------------------- teardown -------------------------------------
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

template <bool A_MN, bool B_MN>
void launch_variant(const GemmArgs& a, const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmC,
                    const CUtensorMap& tmD, const KParams& p, int grid) {
  static PerDeviceOnce once;
  bool& configured = once.current();
  auto kern = gemm_bf16_kernel<A_MN, B_MN>;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) throw std::runtime_error(std::string("gemm: cannot raise shared memory limit: ") + cudaGetErrorString(e));
    configured = true;
  }
  kern<<<grid, NUM_THREADS, SMEM_BYTES, a.stream>>>(tmA, tmB, tmC, tmD, p);
}

}  // namespace

void launch_gemm_bf16(const GemmArgs& a) {
  if (a.M <= 0 || a.N <= 0 || a.K <= 0) return;
  if (a.N % 8 != 0 || a.K % 8 != 0) throw std::runtime_error("gemm_bf16: N and K must be multiples of 8");
  if (a.a_mn && a.M % 8 != 0) throw std::runtime_error("gemm_bf16: M must be a multiple of 8 for a transposed A");
  if (a.lda % 8 != 0 || a.ldb % 8 != 0 || a.ldc % (a.out_fp32 ? 4 : 8) != 0)
    throw std::runtime_error("gemm_bf16: leading dimensions must keep rows 16-byte aligned");
  if (a.d_mode != 0 && (a.D == nullptr || a.ldd % (a.d_mode == 2 ? 4 : 8) != 0))
    throw std::runtime_error("gemm_bf16: bad addend");
  if (a.pull_bytes % 16 != 0 || (a.pull_bytes != 0 && (a.pull_src == nullptr || a.pull_dst == nullptr)))
    throw std::runtime_error("gemm_bf16: the pulled range must be a multiple of 16 bytes with both ends given");
  if (a.scatter_ranks != 0) {
    if (a.scatter_ranks < 1 || a.scatter_ranks > 8 || a.scatter_rows_per_rank <= 0 ||
        a.scatter_rows_per_rank * a.scatter_ranks < a.M || a.ldc % 8 != 0 || a.out_fp32 || a.scatter_src_rank < 0 ||
        a.scatter_src_rank >= a.scatter_ranks)
      throw std::runtime_error("gemm_bf16: bad scatter description");
    for (int r = 0; r < a.scatter_ranks; ++r)
      if (a.scatter_base[r] == nullptr) throw std::runtime_error("gemm_bf16: missing scatter base");
  }

  // K-major operand: global [rows, K]; box 64 (K) x rows-per-tile.
  // MN-major operand: global [K, rows]; box 64 (rows) x 64 (K), several boxes per stage.
  CUtensorMap tmA = a.a_mn ? make_tma_2d(a.A, 2, (uint64_t)a.K, (uint64_t)a.M, (uint64_t)a.lda, 64, BK)
                           : make_tma_2d(a.A, 2, (uint64_t)a.M, (uint64_t)a.K, (uint64_t)a.lda, BK, BM);
  CUtensorMap tmB = a.b_mn ? make_tma_2d(a.B, 2, (uint64_t)a.K, (uint64_t)a.N, (uint64_t)a.ldb, 64, BK)
                           : make_tma_2d(a.B, 2, (uint64_t)a.N, (uint64_t)a.K, (uint64_t)a.ldb, BK, BN);
  KParams p;
  p.M = a.M; p.N = a.N; p.K = a.K;
  p.ldc = a.ldc; p.ldd = a.ldd;
  p.C = a.C; p.D = a.D;
  p.out_fp32 = a.out_fp32; p.d_mode = a.d_mode;
  p.tma_store = (!a.out_fp32 && a.d_mode != 2 && a.scatter_ranks == 0) ? 1 : 0;
  // box: 64 columns (one 128-byte swizzle span) x the 32 rows of one epilogue warp
  CUtensorMap tmC = p.tma_store ? make_tma_2d(a.C, 2, (uint64_t)a.M, (uint64_t)a.N, (uint64_t)a.ldc, 64, 32) : tmA;
  CUtensorMap tmD = (p.tma_store && a.d_mode == 1) ? make_tma_2d(a.D, 2, (uint64_t)a.M, (uint64_t)a.N, (uint64_t)a.ldd, 64, 32) : tmA;
  p.num_m = (a.M + BM - 1) / BM;
  p.num_n = (a.N + BN - 1) / BN;
  p.pull_src = reinterpret_cast<const uint4*>(a.pull_src);
  p.pull_dst = reinterpret_cast<uint4*>(a.pull_dst);
  p.pull_nvec = a.pull_bytes / 16;
  p.scatter_ranks = a.scatter_ranks;
  p.scatter_rows_per_rank = a.scatter_rows_per_rank;
  p.scatter_src_rank = a.scatter_src_rank;
  for (int r = 0; r < 8; ++r) p.scatter_base[r] = reinterpret_cast<__nv_bfloat16*>(a.scatter_base[r]);
  p.status = a.status;
  const int tiles = p.num_m * p.num_n;
  const int grid = tiles < a.sm_count ? tiles : a.sm_count;
  if (a.a_mn) {
    if (a.b_mn) launch_variant<true, true>(a, tmA, tmB, tmC, tmD, p, grid);
    else launch_variant<true, false>(a, tmA, tmB, tmC, tmD, p, grid);
  } else {
    if (a.b_mn) launch_variant<false, true>(a, tmA, tmB, tmC, tmD, p, grid);
    else launch_variant<false, false>(a, tmA, tmB, tmC, tmD, p, grid);
  }
}

}  // namespace zx
