// Microbenchmark: issue rate of tcgen05.mma shapes from one CTA. Zero operands; bounded waits.
#include <cstdio>
#include "../common/ptx.cuh"
using namespace zx;
template <int mode, int IL>
__global__ void __launch_bounds__(128) mma_rate(int reps, long long* out, int* abort_flag) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  __shared__ uint64_t bar;
  __shared__ uint32_t tmem_base_s;
  uint4* z = (uint4*)smem;
  for (int i = threadIdx.x; i < (96 * 1024) / 16; i += 128) z[i] = make_uint4(0, 0, 0, 0);
  if (threadIdx.x == 0) { mbar_init(&bar, 1); fence_mbar_init(); }
  fence_proxy_async_smem();
  __syncthreads();
  if (threadIdx.x < 32) { tmem_alloc(&tmem_base_s, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  uint32_t t = tmem_base_s;
  if (threadIdx.x < 32) {
    uint32_t a_addr = smem_u32(smem), b_addr = smem_u32(smem + 32 * 1024);
    int N = (mode == 1) ? 256 : (mode == 5 ? 64 : 128);
    bool ts = (mode == 2 || mode == 3);
    bool b_mn = (mode == 2 || mode == 4);
    uint32_t idesc = make_idesc(128, N, 1, 1, 0, b_mn ? 1 : 0);
    uint64_t a_desc = make_smem_desc_sw128(a_addr, 0, 1024);
    uint64_t b_desc = b_mn ? make_smem_desc_sw128(b_addr, 16384, 1024) : make_smem_desc_sw128(b_addr, 0, 1024);
    uint32_t b_chunk = (uint32_t)N * 128;  // K-major: bytes per 64-wide K chunk
    __syncwarp();
    long long t0 = clock64();
    for (int r = 0; r < reps; ++r) {
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        uint32_t d = (IL == 1) ? t + (k & 1) * 256 : (IL == 2 ? t + (k & 3) * 128 : t + (r & 1) * 256);
        if (IL == 3) d = t;
        uint64_t bd = b_mn ? desc_advance(b_desc, k * 2048) : desc_advance(b_desc, (k >> 2) * b_chunk + (k & 3) * 32);
        if (ts) umma_ts_w(d, t + 384 + (k >> 2) * 32 + (k & 3) * 8, bd, idesc, (IL == 1 ? k > 1 : (IL == 2 ? k > 3 : k > 0)));
        else umma_ss_w(d, desc_advance(a_desc, (k >> 2) * 16384 + (k & 3) * 32), bd, idesc, (IL == 1 ? k > 1 : (IL == 2 ? k > 3 : k > 0)));
      }
    }
    long long t1 = clock64();
    umma_commit_w(&bar);
    bool ok = mbar_wait_w(&bar, 0, abort_flag);
    long long t2 = clock64();
    if (threadIdx.x == 0 && blockIdx.x == 0) { out[0] = t1 - t0; out[1] = t2 - t0; out[2] = ok; }
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x < 32) tmem_dealloc(t, 512);
}

template <int mode, int IL>
void run(const char* name, long long* out, int* flag) {
  cudaFuncSetAttribute(mma_rate<mode, IL>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
  long long h[3];
  for (int it = 0; it < 2; ++it) {
    mma_rate<mode, IL><<<1, 128, 100 * 1024>>>(64, out, flag);
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) { printf("error %s\n", cudaGetErrorString(e)); exit(1); }
  }
  cudaMemcpy(h, out, 24, cudaMemcpyDeviceToHost);
  printf("%-44s issue %6lld clk  done %6lld clk  -> %.1f clk / instr ok=%lld\n", name, h[0], h[1], h[1] / 512.0, h[2]);
}
int main() {
  long long* out; int* flag;
  cudaMalloc(&out, 64); cudaMalloc(&flag, 4); cudaMemset(flag, 0, 4);
  run<0, 0>("SS N=128 Kmaj, one chain per 8", out, flag);
  run<0, 3>("SS N=128 Kmaj, same D always", out, flag);
  run<0, 1>("SS N=128 Kmaj, 2 chains interleaved", out, flag);
  run<0, 2>("SS N=128 Kmaj, 4 chains interleaved", out, flag);
  run<5, 0>("SS N=64 Kmaj, one chain", out, flag);
  run<5, 2>("SS N=64 Kmaj, 4 chains", out, flag);
  run<1, 0>("SS N=256 Kmaj, one chain", out, flag);
  run<2, 0>("TS N=128 MNmaj, one chain", out, flag);
  run<2, 1>("TS N=128 MNmaj, 2 chains", out, flag);
  run<4, 0>("SS N=128 MNmaj, one chain", out, flag);
  return 0;
}
