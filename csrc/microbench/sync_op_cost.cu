// Cost of individual synchronisation instructions, one warp, nothing else running.
#include <cstdio>
#include "../common/ptx.cuh"
using namespace zx;
__global__ void __launch_bounds__(128) opcost(long long* out, int* abort_flag) {
  __shared__ uint64_t bar, bar2;
  __shared__ uint32_t tmem_base_s;
  if (threadIdx.x == 0) { mbar_init(&bar, 1); mbar_init(&bar2, 4); fence_mbar_init(); }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (warp == 0) { tmem_alloc(&tmem_base_s, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  uint32_t t = tmem_base_s + ((uint32_t)(warp * 32) << 16);
  if (threadIdx.x == 0) mbar_arrive(&bar);   // phase 0 complete
  __syncthreads();
  long long c[16];
  uint32_t r[32];
  for (int rep = 0; rep < 2; ++rep) {
    c[0] = clock64();
    bool ok = mbar_try_wait(&bar, 0);
    c[1] = clock64();
    ok = __all_sync(0xffffffffu, ok);
    c[2] = clock64();
    tc_fence_after();
    c[3] = clock64();
    tmem_ld_32x32b_x32(t, r);
    tmem_wait_ld();
    c[4] = clock64();
#pragma unroll
    for (int i = 0; i < 32; ++i) r[i] += ok;
    tmem_st_32x32b_x32(t + 32, r);
    tmem_wait_st();
    c[5] = clock64();
    tc_fence_before();
    c[6] = clock64();
    mbar_arrive_warp(&bar2);
    c[7] = clock64();
    ok = mbar_wait(&bar, 0, abort_flag);
    c[8] = clock64();
    (void)ok;
    c[9] = clock64();
  }
  if (threadIdx.x == 32 && blockIdx.x == 0) for (int i = 0; i < 10; ++i) out[i] = c[i] - c[0];
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base_s, 512);
}
int main() {
  long long* out; int* flag;
  cudaMalloc(&out, 512); cudaMalloc(&flag, 4); cudaMemset(flag, 0, 4);
  opcost<<<1, 128>>>(out, flag);
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) { printf("error %s\n", cudaGetErrorString(e)); return 1; }
  long long h[16];
  cudaMemcpy(h, out, 128, cudaMemcpyDeviceToHost);
  const char* n[] = {"start", "try_wait(done)", "all_sync", "fence::after", "tmem ld x32+wait", "add + tmem st x32+wait",
                     "fence::before", "arrive_warp", "mbar_wait(done)", "-"};
  for (int i = 1; i < 9; ++i) printf("%-24s %lld clk\n", n[i], h[i] - h[i - 1]);
  return 0;
}
