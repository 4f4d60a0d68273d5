// MMA rate under concurrent TMEM ld/st traffic and bulk global->smem copies.
#include <cstdio>
#include <cstdlib>
#include "../common/ptx.cuh"
using namespace zx;
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
// warps: 0 = MMA, 1 = bulk copier, 2..9 = TMEM ld/st traffic
template <int TS, int LOAD>
__global__ void __launch_bounds__(320) mma_load(int reps, const uint8_t* gsrc, long long* out, int* abort_flag) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  __shared__ uint64_t bar, cbar;
  __shared__ uint32_t tmem_base_s;
  __shared__ volatile int done;
  uint4* z = (uint4*)smem;
  for (int i = threadIdx.x; i < (64 * 1024) / 16; i += blockDim.x) z[i] = make_uint4(0, 0, 0, 0);
  if (threadIdx.x == 0) { mbar_init(&bar, 1); mbar_init(&cbar, 1); done = 0; fence_mbar_init(); }
  fence_proxy_async_smem();
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (warp == 0) { tmem_alloc(&tmem_base_s, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  uint32_t t = tmem_base_s;
  if (warp == 0) {
    uint32_t a_addr = smem_u32(smem), b_addr = smem_u32(smem + 32 * 1024);
    constexpr uint32_t idesc = make_idesc(128, 128, 1, 1, 0, TS ? 1 : 0);
    uint64_t a_desc = make_smem_desc_sw128(a_addr, 0, 1024);
    uint64_t b_desc = TS ? make_smem_desc_sw128(b_addr, 16384, 1024) : make_smem_desc_sw128(b_addr, 0, 1024);
    __syncwarp();
    long long t0 = clock64();
    for (int r = 0; r < reps; ++r) {
      uint32_t d = t + (r & 1) * 128;
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        uint64_t bd = TS ? desc_advance(b_desc, k * 2048) : desc_advance(b_desc, (k >> 2) * 16384 + (k & 3) * 32);
        if (TS) umma_ts_w(d, t + 256 + (k >> 2) * 32 + (k & 3) * 8, bd, idesc, k > 0);
        else umma_ss_w(d, desc_advance(a_desc, (k >> 2) * 16384 + (k & 3) * 32), bd, idesc, k > 0);
      }
    }
    umma_commit_w(&bar);
    bool ok = mbar_wait_w(&bar, 0, abort_flag);
    long long t2 = clock64();
    if (lane == 0) { done = 1; if (blockIdx.x == 0) { out[0] = t2 - t0; out[2] = ok; } }
  } else if (warp == 1) {
    long long n = 0;
    if ((LOAD & 2) && lane == 0) {
      uint8_t* dst = smem + 64 * 1024;
      uint32_t ph = 0;
      while (!done && n < 100000) {
        mbar_expect_tx(&cbar, 64 * 1024);
        for (int i = 0; i < 4; ++i)
          bulk_g2s(dst + i * 16384, gsrc + ((size_t)blockIdx.x * 4 + i) * 16384, 16384, &cbar);
        if (!mbar_wait(&cbar, ph, abort_flag)) break;
        ph ^= 1; ++n;
      }
      if (blockIdx.x == 0) out[1] = n;
    }
  } else {
    long long n = 0;
    if (LOAD & 1) {
      uint32_t r[32];
      uint32_t ta = t + 320 + ((uint32_t)(warp & 3) * 32 << 16) + ((warp - 2) >> 2) * 64;
      while (!done && n < 1000000) {
        tmem_ld_32x32b_x32(ta, r);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) r[i] += 1;
        tmem_st_32x32b_x32(ta + 32, r);
        tmem_wait_st();
        ++n;
      }
      if (threadIdx.x == 64 && blockIdx.x == 0) out[3] = n;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(t, 512);
}
template <int TS, int LOAD>
void run(const char* name, const uint8_t* g, long long* out, int* flag) {
  cudaFuncSetAttribute(mma_load<TS, LOAD>, cudaFuncAttributeMaxDynamicSharedMemorySize, 140 * 1024);
  long long h[4];
  for (int it = 0; it < 2; ++it) {
    cudaMemset(out, 0, 64);
    mma_load<TS, LOAD><<<148, 320, 140 * 1024>>>(64, g, out, flag);
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) { printf("error %s\n", cudaGetErrorString(e)); exit(1); }
  }
  cudaMemcpy(h, out, 32, cudaMemcpyDeviceToHost);
  printf("%-40s %.1f clk / mma instr   bulk 64KB batches %lld (%.1f B/clk)  tmem ld+st rounds/warp %lld  ok=%lld\n", name,
         h[0] / 512.0, h[1], h[1] * 65536.0 / h[0], h[3], h[2]);
}
int main() {
  long long* out; int* flag; uint8_t* g;
  cudaMalloc(&out, 64); cudaMalloc(&flag, 4); cudaMemset(flag, 0, 4);
  cudaMalloc(&g, 148 * 65536); cudaMemset(g, 0, 148 * 65536);
  run<0, 0>("SS alone", g, out, flag);
  run<0, 1>("SS + tmem ld/st (8 warps)", g, out, flag);
  run<0, 2>("SS + bulk copies", g, out, flag);
  run<0, 3>("SS + both", g, out, flag);
  run<1, 0>("TS alone", g, out, flag);
  run<1, 1>("TS + tmem ld/st (8 warps)", g, out, flag);
  run<1, 2>("TS + bulk copies", g, out, flag);
  run<1, 3>("TS + both", g, out, flag);
  return 0;
}
