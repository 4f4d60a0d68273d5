// How late do waiters observe a tcgen05.commit on an mbarrier, by number of waiting warps and wait length.
#include <cstdio>
#include <cstdlib>
#include "../common/ptx.cuh"
using namespace zx;
// warp 0 = MMA issuer; warps 1..NW = waiters (all lanes wait, like the attention kernels)
__global__ void __launch_bounds__(544) wake(int nw, int reps, long long* out, int* abort_flag) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  __shared__ uint64_t bar;
  __shared__ uint32_t tmem_base_s;
  uint4* z = (uint4*)smem;
  for (int i = threadIdx.x; i < (64 * 1024) / 16; i += blockDim.x) z[i] = make_uint4(0, 0, 0, 0);
  if (threadIdx.x == 0) { mbar_init(&bar, 1); fence_mbar_init(); }
  fence_proxy_async_smem();
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (warp == 0) { tmem_alloc(&tmem_base_s, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  uint32_t t = tmem_base_s;
  long long t0 = clock64();
  if (warp == 0) {
    uint32_t a_addr = smem_u32(smem), b_addr = smem_u32(smem + 32 * 1024);
    constexpr uint32_t idesc = make_idesc(128, 128, 1, 1, 0, 0);
    uint64_t a_desc = make_smem_desc_sw128(a_addr, 0, 1024);
    uint64_t b_desc = make_smem_desc_sw128(b_addr, 0, 1024);
    for (int r = 0; r < reps; ++r) {
#pragma unroll
      for (int k = 0; k < 8; ++k)
        umma_ss_w(t, desc_advance(a_desc, (k >> 2) * 16384 + (k & 3) * 32),
                  desc_advance(b_desc, (k >> 2) * 16384 + (k & 3) * 32), idesc, k > 0);
    }
    umma_commit_w(&bar);
    bool ok = mbar_wait_w(&bar, 0, abort_flag);
    long long t1 = clock64();
    if (lane == 0 && blockIdx.x == 0) { out[0] = t1 - t0; out[63] = ok; }
  } else if (warp <= nw) {
    bool ok = mbar_wait(&bar, 0, abort_flag);
    ok = __all_sync(0xffffffffu, ok);
    long long t1 = clock64();
    if (lane == 0 && blockIdx.x == 0) out[warp] = t1 - t0;
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(t, 512);
}
int main() {
  long long* out; int* flag;
  cudaMalloc(&out, 512); cudaMalloc(&flag, 4); cudaMemset(flag, 0, 4);
  cudaFuncSetAttribute(wake, cudaFuncAttributeMaxDynamicSharedMemorySize, 70 * 1024);
  for (int reps : {1, 2, 4, 8}) for (int nw : {1, 4, 8, 16}) {
    long long h[64];
    for (int it = 0; it < 2; ++it) {
      cudaMemset(out, 0, 512);
      wake<<<148, 544, 70 * 1024>>>(nw, reps, out, flag);
      cudaError_t e = cudaDeviceSynchronize();
      if (e != cudaSuccess) { printf("error %s\n", cudaGetErrorString(e)); return 1; }
    }
    cudaMemcpy(h, out, 512, cudaMemcpyDeviceToHost);
    printf("mma groups %d (%d clk ideal) waiters %2d: issuer sees %5lld; waiters see", reps, reps * 512, nw, h[0]);
    long long mx = 0;
    for (int w = 1; w <= nw; ++w) { if (nw <= 8 || w % 2 == 0) printf(" %lld", h[w]); if (h[w] > mx) mx = h[w]; }
    printf("  (max lag %lld)\n", mx - h[0]);
  }
  return 0;
}
