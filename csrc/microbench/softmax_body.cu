// Cost of the forward softmax body (one 128-column row per thread) for W warps on one SM, nothing else running.
#include <cstdio>
#include "../common/ptx.cuh"
using namespace zx;
constexpr float NEG_BIG = -1e30f;
__device__ __forceinline__ float fmax3_(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
// V bit0: fmax3; bit1: packed sum; bits 2-4: polynomial share in eighths
template <int V>
__global__ void __launch_bounds__(352) softmax_cost(int nwarps, int reps, long long* out, float* sink, float scale_log2, int spin_mode = 0) {
  __shared__ uint32_t tmem_base_s;
  __shared__ uint64_t never;
  __shared__ volatile int done_cnt;
  if (threadIdx.x == 0) { mbar_init(&never, 1); fence_mbar_init(); done_cnt = 0; }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (warp == 0) { tmem_alloc(&tmem_base_s, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t s_tmem = tmem_base_s + ((uint32_t)((warp & 3) * 32) << 16) + (warp >> 2) * 128;
  if (warp < nwarps) {
    float m_used = NEG_BIG, l = 0.f;
    long long t0 = 0, t_ld = 0, t_end = 0, acc_ld = 0, acc_all = 0;
    for (int it = 0; it < reps; ++it) {
      t0 = clock64();
      uint32_t sr[128];
      tmem_ld_32x32b_x32(s_tmem + 0, sr);
      tmem_ld_32x32b_x32(s_tmem + 32, sr + 32);
      tmem_ld_32x32b_x32(s_tmem + 64, sr + 64);
      tmem_ld_32x32b_x32(s_tmem + 96, sr + 96);
      tmem_wait_ld();
      t_ld = clock64();
      float mx4[4] = {NEG_BIG, NEG_BIG, NEG_BIG, NEG_BIG};
      if (V & 1) {
#pragma unroll
        for (int c = 0; c < 128; c += 8) {
          mx4[0] = fmax3_(mx4[0], __uint_as_float(sr[c + 0]), __uint_as_float(sr[c + 1]));
          mx4[1] = fmax3_(mx4[1], __uint_as_float(sr[c + 2]), __uint_as_float(sr[c + 3]));
          mx4[2] = fmax3_(mx4[2], __uint_as_float(sr[c + 4]), __uint_as_float(sr[c + 5]));
          mx4[3] = fmax3_(mx4[3], __uint_as_float(sr[c + 6]), __uint_as_float(sr[c + 7]));
        }
      } else {
#pragma unroll
        for (int c = 0; c < 128; ++c) mx4[c & 3] = fmaxf(mx4[c & 3], __uint_as_float(sr[c]));
      }
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      const float m_cur = mx * scale_log2;
      if (it == 0 || m_cur > m_used + 8.f) { l *= fast_exp2(m_used - m_cur); m_used = m_cur; }
      uint32_t pk[64];
      float sum4[4] = {0.f, 0.f, 0.f, 0.f};
      const float2 sl2 = make_float2(scale_log2, scale_log2);
      const float2 nm2 = make_float2(-m_used, -m_used);
#pragma unroll
      for (int c = 0; c < 64; ++c) {
        const float2 x = __ffma2_rn(make_float2(__uint_as_float(sr[2 * c]), __uint_as_float(sr[2 * c + 1])), sl2, nm2);
        constexpr int PS = (V >> 2) & 7;   // eighths
        const bool poly = PS == 2 ? (c & 3) == 3 : (c & 7) < PS;   // a quarter: every fourth pair
        float2 pe;
        if (poly) pe = exp2_poly2(x); else pe = make_float2(fast_exp2(x.x), fast_exp2(x.y));
        if (V & 2) { const float2 a2 = __fadd2_rn(make_float2(sum4[c & 1], sum4[2 + (c & 1)]), pe); sum4[c & 1] = a2.x; sum4[2 + (c & 1)] = a2.y; }
        else sum4[c & 3] += pe.x + pe.y;
        pk[c] = pack_bf16x2(pe.x, pe.y);
      }
      l += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
      tmem_st_32x32b_x32(s_tmem + 0, pk);
      tmem_st_32x32b_x32(s_tmem + 32, pk + 32);
      tmem_wait_st();
      t_end = clock64();
      if (it > 0) { acc_ld += t_ld - t0; acc_all += t_end - t0; }
    }
    if (lane == 0) { out[warp * 2] = acc_ld / (reps - 1); out[warp * 2 + 1] = acc_all / (reps - 1); }
    sink[threadIdx.x] = l + m_used;
    __syncwarp();
    if (lane == 0) atomicAdd((int*)&done_cnt, 1);
  } else if (spin_mode && warp < nwarps + 4) {
    // a waiting neighbour: polls a barrier nobody completes until the working warps are done (bounded)
    int guard = 0;
    while (done_cnt < nwarps && guard < 2000000) {
      if (spin_mode == 1) { for (int i = 0; i < 16; ++i) if (mbar_try_wait(&never, 0)) break; }
      else { if (!mbar_try_wait(&never, 0)) __nanosleep(spin_mode); }
      ++guard;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base_s, 512);
}

template <int V>
void run(const char* name, long long* out, float* sink) {
  for (int nw : {4, 8}) {   // one or two working warps per scheduler
    cudaMemset(out, 0, 512);
    softmax_cost<V><<<1, 352>>>(nw, 9, out, sink, 0.1275f, 0);
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) { printf("error %s\n", cudaGetErrorString(e)); exit(1); }
    long long h[32];
    cudaMemcpy(h, out, 256, cudaMemcpyDeviceToHost);
    printf("%-40s %d warps: clk per 128x128 tile per warp: %lld\n", name, nw, h[1]);
  }
}
template <int V>
void run_with_waiters(const char* name, long long* out, float* sink) {
  for (int spin : {0, 1, 32, 200}) {   // 0: nobody waits; 1: try_wait polling; else test + nanosleep(n)
    cudaMemset(out, 0, 512);
    softmax_cost<V><<<1, 352>>>(4, 9, out, sink, 0.1275f, spin);
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) { printf("error %s\n", cudaGetErrorString(e)); exit(1); }
    long long h[32];
    cudaMemcpy(h, out, 256, cudaMemcpyDeviceToHost);
    printf("%-24s 4 working warps + 4 waiting (mode %3d): clk per tile per warp: %lld\n", name, spin, h[1]);
  }
}
int main() {
  long long* out; float* sink;
  cudaMalloc(&out, 512); cudaMalloc(&sink, 4096);
  run<0>("scalar row sum (two adds per pair)", out, sink);
  run<1>("three-input maxima", out, sink);
  run<2>("packed row sum", out, sink);
  run<2 + 4 * 1>("packed sum + 1/8 polynomial exp2", out, sink);
  run<2 + 4 * 2>("packed sum + 1/4 polynomial exp2", out, sink);
  run<2 + 4 * 4>("packed sum + 1/2 polynomial exp2", out, sink);
  run_with_waiters<2>("packed row sum", out, sink);
  return 0;
}
