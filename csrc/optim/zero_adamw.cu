// Reduce-scatter + AdamW + all-gather in one kernel over NVLink peer memory.
//
// Each rank owns a contiguous shard of the flat parameter space. For every 4 elements of its shard
// a thread (1) loads the fp32 gradients of that range from every rank's gradient buffer with P2P
// loads and sums them (the reduce-scatter), (2) applies the scale / clip factor and the AdamW
// update to its fp32 master weight (kept as bf16 high half + int16 remainder), and (3) stores the
// new bf16 parameter into every rank's parameter buffer with P2P stores (the all-gather). No
// intermediate buffer, no NCCL. The two halves can also run as separate launches (reduce, then
// update) when a global gradient norm is needed in between.
// The reference does this as bucketed all-reduce + copy-back + torch AdamW
// (zenyx/runtime/scheduler.py:32-107,158-160).
#include "../common/ptx.cuh"
#include "zero.h"

namespace zx {

namespace {

struct ZParams {
  PeerPtrs grads, params;
  int nranks, rank;
  size_t shard_begin, n_shard, decay_end;
  float* g_shard;
  int16_t* p_lo;
  void* m;
  void* v;
  float* sumsq;
  const float* clip_coef;
  int do_reduce, do_update, zero_grads;
  float grad_scale, lr, beta1, beta2, eps, weight_decay, bias1, bias2;
};

// NR: number of ranks known at compile time (1, 2, 4, 8), so the peer loads of one element are all in
// flight together instead of one NVLink round trip after another; 0 = any count, loop at run time.
//
// Memory behaviour: per parameter the step moves 32 bytes through five streams of 8 or 16 bytes per thread. One
// float4 group per thread per loop trip left the kernel at 0.23 of the copy rate: too few bytes in flight per SM for
// HBM latency, and the loads sat behind `asm volatile` statements that the compiler may not reorder. Each thread now
// handles UNROLL groups per trip, issues ALL of their loads (through the __ldcs intrinsic, which the compiler can
// schedule) before the first dependent instruction, and the grid is sized to the work instead of capped.
constexpr int ZERO_UNROLL = 2;

struct Group {   // one float4 group of every stream
  float4 g, mm, vv;
  uint2 hi, lo;
};

// Adam's moments in memory: fp32, or bf16 (SB) to halve their footprint; the arithmetic is fp32 either way.
template <bool SB>
__device__ __forceinline__ float4 ld_state(const void* base, size_t i) {
  if constexpr (SB) {
    const uint2 u = reinterpret_cast<const uint2*>(base)[i];
    const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y);
    return make_float4(a.x, a.y, b.x, b.y);
  } else {
    return reinterpret_cast<const float4*>(base)[i];
  }
}
template <bool SB>
__device__ __forceinline__ void st_state(void* base, size_t i, const float* x) {
  if constexpr (SB)
    reinterpret_cast<uint2*>(base)[i] = make_uint2(pack_bf16x2(x[0], x[1]), pack_bf16x2(x[2], x[3]));
  else
    reinterpret_cast<float4*>(base)[i] = make_float4(x[0], x[1], x[2], x[3]);
}

template <int NR, bool SB>
__global__ void __launch_bounds__(256) zero_step_kernel(ZParams p) {
  __shared__ float s_red[8];
  const size_t nvec = p.n_shard >> 2;
  float local_ss = 0.f;
  const float clip = (p.do_update && p.clip_coef != nullptr) ? *p.clip_coef : 1.f;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  uint16_t* own_params = reinterpret_cast<uint16_t*>(p.params.p[p.rank]);
  for (size_t i0 = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i0 < nvec; i0 += stride * ZERO_UNROLL) {
    Group u[ZERO_UNROLL];
    bool live[ZERO_UNROLL];
    // ---- all loads of this trip ----
#pragma unroll
    for (int q = 0; q < ZERO_UNROLL; ++q) {
      const size_t i = i0 + (size_t)q * stride;
      live[q] = i < nvec;
      if (!live[q]) continue;
      const size_t gi = p.shard_begin + (i << 2);  // global element index
      if (p.do_reduce) {
        float4 g = make_float4(0.f, 0.f, 0.f, 0.f);
        // start with the next rank so the R readers of one step hit R different owners
        if constexpr (NR > 0) {
          float4 a[NR];
#pragma unroll
          for (int k = 0; k < NR; ++k) {
            int r = p.rank + 1 + k;
            if (r >= NR) r -= NR;
            a[k] = __ldcs(reinterpret_cast<const float4*>(reinterpret_cast<float*>(p.grads.p[r]) + gi));
          }
#pragma unroll
          for (int k = 0; k < NR; ++k) { g.x += a[k].x; g.y += a[k].y; g.z += a[k].z; g.w += a[k].w; }
        } else {
          for (int k = 0; k < p.nranks; ++k) {
            int r = p.rank + 1 + k;
            if (r >= p.nranks) r -= p.nranks;
            const float4 a = __ldcs(reinterpret_cast<const float4*>(reinterpret_cast<float*>(p.grads.p[r]) + gi));
            g.x += a.x; g.y += a.y; g.z += a.z; g.w += a.w;
          }
        }
        u[q].g = g;
      } else {
        u[q].g = __ldcs(reinterpret_cast<const float4*>(p.g_shard) + i);
      }
      if (p.do_update) {
        u[q].hi = *reinterpret_cast<const uint2*>(own_params + gi);
        u[q].lo = reinterpret_cast<const uint2*>(p.p_lo)[i];
        u[q].mm = ld_state<SB>(p.m, i);
        u[q].vv = ld_state<SB>(p.v, i);
      }
    }
    // ---- arithmetic and stores ----
#pragma unroll
    for (int q = 0; q < ZERO_UNROLL; ++q) {
      if (!live[q]) continue;
      const size_t i = i0 + (size_t)q * stride;
      const size_t gi = p.shard_begin + (i << 2);
      float4 g = u[q].g;
      if (p.do_reduce) {
        if (p.zero_grads) {
          const int nr = NR > 0 ? NR : p.nranks;
          for (int r = 0; r < nr; ++r)
            *reinterpret_cast<float4*>(reinterpret_cast<float*>(p.grads.p[r]) + gi) = make_float4(0.f, 0.f, 0.f, 0.f);
        }
        g.x *= p.grad_scale; g.y *= p.grad_scale; g.z *= p.grad_scale; g.w *= p.grad_scale;
        local_ss += g.x * g.x + g.y * g.y + g.z * g.z + g.w * g.w;
        if (!p.do_update) {   // norm pass: keep the reduced shard if there is room for it, else only its norm
          if (p.g_shard != nullptr) reinterpret_cast<float4*>(p.g_shard)[i] = g;
          continue;
        }
      }
      // ---- AdamW on the split master ----
      g.x *= clip; g.y *= clip; g.z *= clip; g.w *= clip;
      const uint2 hi = u[q].hi, lo = u[q].lo;
      const float4 mm = u[q].mm, vv = u[q].vv;
      const uint16_t h[4] = {(uint16_t)(hi.x & 0xffff), (uint16_t)(hi.x >> 16), (uint16_t)(hi.y & 0xffff), (uint16_t)(hi.y >> 16)};
      const int16_t l[4] = {(int16_t)(lo.x & 0xffff), (int16_t)(lo.x >> 16), (int16_t)(lo.y & 0xffff), (int16_t)(lo.y >> 16)};
      float gr[4] = {g.x, g.y, g.z, g.w};
      float ma[4] = {mm.x, mm.y, mm.z, mm.w};
      float va[4] = {vv.x, vv.y, vv.z, vv.w};
      const float wd = gi < p.decay_end ? p.weight_decay : 0.f;
      uint32_t nh[4], nl[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float w = __uint_as_float(((uint32_t)h[j] << 16) + (uint32_t)(int32_t)l[j]);
        ma[j] = p.beta1 * ma[j] + (1.f - p.beta1) * gr[j];
        va[j] = p.beta2 * va[j] + (1.f - p.beta2) * gr[j] * gr[j];
        w = w * (1.f - p.lr * wd) - p.lr * (ma[j] / p.bias1) / (sqrtf(va[j] / p.bias2) + p.eps);
        const uint32_t bits = __float_as_uint(w);
        const uint32_t hh = (bits + 0x8000u) >> 16;
        nh[j] = hh & 0xffffu;
        nl[j] = (bits - (hh << 16)) & 0xffffu;
      }
      st_state<SB>(p.m, i, ma);
      st_state<SB>(p.v, i, va);
      reinterpret_cast<uint2*>(p.p_lo)[i] = make_uint2(nl[0] | (nl[1] << 16), nl[2] | (nl[3] << 16));
      const uint2 new_hi = make_uint2(nh[0] | (nh[1] << 16), nh[2] | (nh[3] << 16));
      // all-gather: push the new bf16 parameters into every rank's buffer
      for (int r = 0; r < p.nranks; ++r)
        *reinterpret_cast<uint2*>(reinterpret_cast<uint16_t*>(p.params.p[r]) + gi) = new_hi;
    }
  }
  if (p.do_reduce && p.sumsq != nullptr) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) local_ss += __shfl_xor_sync(0xffffffffu, local_ss, o);
    if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = local_ss;
    __syncthreads();
    if (threadIdx.x == 0) {
      float t = 0.f;
      for (int w = 0; w < (int)(blockDim.x >> 5); ++w) t += s_red[w];
      atomicAdd(p.sumsq, t);
    }
  }
}

}  // namespace

void launch_zero_step(const ZeroArgs& a) {
  if (a.n_shard == 0) return;
  ZParams p;
  p.grads = a.grads; p.params = a.params;
  p.nranks = a.nranks; p.rank = a.rank;
  p.shard_begin = a.shard_begin; p.n_shard = a.n_shard; p.decay_end = a.decay_end;
  p.g_shard = a.g_shard; p.p_lo = a.p_lo; p.m = a.m; p.v = a.v;
  p.sumsq = a.sumsq; p.clip_coef = a.clip_coef;
  p.do_reduce = a.do_reduce; p.do_update = a.do_update; p.zero_grads = a.zero_grads;
  p.grad_scale = a.grad_scale; p.lr = a.lr; p.beta1 = a.beta1; p.beta2 = a.beta2; p.eps = a.eps;
  p.weight_decay = a.weight_decay;
  p.bias1 = 1.f - powf(a.beta1, (float)a.step);
  p.bias2 = 1.f - powf(a.beta2, (float)a.step);
  const size_t nvec = a.n_shard / 4;
  size_t blocks = (nvec + 256 * ZERO_UNROLL - 1) / (256 * ZERO_UNROLL);
  const size_t cap = (size_t)a.sm_count * 64;   // several waves: the tail of one hides under the head of the next
  if (blocks > cap) blocks = cap;
  const unsigned nb = (unsigned)blocks;
#define ZX_ZERO_LAUNCH(NR)                                                            \
  do {                                                                                \
    if (a.state_bf16) zero_step_kernel<NR, true><<<nb, 256, 0, a.stream>>>(p);        \
    else zero_step_kernel<NR, false><<<nb, 256, 0, a.stream>>>(p);                    \
  } while (0)
  switch (a.nranks) {
    case 1: ZX_ZERO_LAUNCH(1); break;
    case 2: ZX_ZERO_LAUNCH(2); break;
    case 4: ZX_ZERO_LAUNCH(4); break;
    case 8: ZX_ZERO_LAUNCH(8); break;
    default: ZX_ZERO_LAUNCH(0); break;
  }
#undef ZX_ZERO_LAUNCH
}

}  // namespace zx
