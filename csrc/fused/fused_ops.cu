// Bandwidth-bound kernels of the Llama block and the optimizer for sm_100a: RMSNorm, RoPE,
// SwiGLU, embedding, softmax cross-entropy, e4m3 KV quantisation, AdamW with a split fp32 master.
// All tensors are bf16 with fp32 math; every access is a 16-byte vector.
#include <cuda_fp8.h>
#include "../common/ptx.cuh"
#include "fused_ops.h"

namespace zx {

namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

__device__ __forceinline__ void unpack8(const uint4& u, float* f) {
  float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
__device__ __forceinline__ uint4 pack8(const float* f) {
  uint4 u;
  u.x = pack_bf16x2(f[0], f[1]);
  u.y = pack_bf16x2(f[2], f[3]);
  u.z = pack_bf16x2(f[4], f[5]);
  u.w = pack_bf16x2(f[6], f[7]);
  return u;
}

// ------------------------------------------------------------------------------------------
// RMSNorm: one warp per row, two passes over a row that stays in L1.
// ------------------------------------------------------------------------------------------
__global__ void rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                   __nv_bfloat16* __restrict__ y, float* __restrict__ rstd, int rows, int H,
                                   float eps) {
  const int warps_per_block = blockDim.x >> 5;
  const int row = blockIdx.x * warps_per_block + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)row * H);
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  uint4* yr = reinterpret_cast<uint4*>(y + (size_t)row * H);
  const int nvec = H >> 3;
  float ss = 0.f;
  for (int i = lane; i < nvec; i += 32) {
    float f[8];
    unpack8(xr[i], f);
#pragma unroll
    for (int j = 0; j < 8; ++j) ss += f[j] * f[j];
  }
  ss = warp_sum(ss);
  const float r = rsqrtf(ss / (float)H + eps);
  if (lane == 0 && rstd != nullptr) rstd[row] = r;
  for (int i = lane; i < nvec; i += 32) {
    float f[8], g[8];
    unpack8(xr[i], f);
    unpack8(wr[i], g);
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = f[j] * r * g[j];
    yr[i] = pack8(f);
  }
}


// Same, for rows of 32 * VPL vectors: the row is loaded once, all loads of a lane in flight together, and
// stays in registers between the sum of squares and the scaling.
template <int VPL>
__global__ void __launch_bounds__(128, 3) rmsnorm_fwd_regs_kernel(const __nv_bfloat16* __restrict__ x,
                                                               const __nv_bfloat16* __restrict__ w,
                                                               __nv_bfloat16* __restrict__ y, float* __restrict__ rstd,
                                                               int rows, float eps) {
  constexpr int H = VPL * 32 * 8;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)row * H);
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  uint4* yr = reinterpret_cast<uint4*>(y + (size_t)row * H);
  uint4 v[VPL];
#pragma unroll
  for (int k = 0; k < VPL; ++k) v[k] = __ldcs(xr + lane + 32 * k);
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < VPL; ++k) {
    float f[8];
    unpack8(v[k], f);
#pragma unroll
    for (int j = 0; j < 8; ++j) ss += f[j] * f[j];
  }
  ss = warp_sum(ss);
  const float r = rsqrtf(ss / (float)H + eps);
  if (lane == 0 && rstd != nullptr) rstd[row] = r;
#pragma unroll
  for (int k = 0; k < VPL; ++k) {
    float f[8], g[8];
    unpack8(v[k], f);
    unpack8(__ldg(wr + lane + 32 * k), g);
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = f[j] * r * g[j];
    yr[lane + 32 * k] = pack8(f);
  }
}

// dx = rstd * (dy*w - xhat * mean(dy*w*xhat)); dw += sum_rows dy * xhat (fp32 atomics per block).
__global__ void rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                                   const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd,
                                   const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dx,
                                   float* __restrict__ dw_accum, int rows, int H) {
  extern __shared__ float s_dw[];  // [H]
  for (int i = threadIdx.x; i < H; i += blockDim.x) s_dw[i] = 0.f;
  __syncthreads();
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  const int nvec = H >> 3;
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  for (int row = blockIdx.x * warps_per_block + (threadIdx.x >> 5); row < rows; row += gridDim.x * warps_per_block) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)row * H);
    const uint4* dyr = reinterpret_cast<const uint4*>(dy + (size_t)row * H);
    uint4* dxr = reinterpret_cast<uint4*>(dx + (size_t)row * H);
    const float r = rstd[row];
    float dot = 0.f;
    for (int i = lane; i < nvec; i += 32) {
      float fx[8], fd[8], fw[8];
      unpack8(xr[i], fx);
      unpack8(dyr[i], fd);
      unpack8(wr[i], fw);
#pragma unroll
      for (int j = 0; j < 8; ++j) dot += fd[j] * fw[j] * fx[j] * r;
    }
    dot = warp_sum(dot) / (float)H;
    for (int i = lane; i < nvec; i += 32) {
      float fx[8], fd[8], fw[8], o[8];
      unpack8(xr[i], fx);
      unpack8(dyr[i], fd);
      unpack8(wr[i], fw);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float xh = fx[j] * r;
        o[j] = r * (fd[j] * fw[j] - xh * dot);
        atomicAdd(&s_dw[i * 8 + j], fd[j] * xh);
      }
      if (dres != nullptr) {  // gradient arriving through the residual branch
        float fr[8];
        unpack8(reinterpret_cast<const uint4*>(dres + (size_t)row * H)[i], fr);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] += fr[j];
      }
      dxr[i] = pack8(o);
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < H; i += blockDim.x) atomicAdd(&dw_accum[i], s_dw[i]);
}


// Same result for rows of up to 512 * VPT vectors, one block of 512 threads per group of R rows: thread i owns
// vectors i, i + 512, ... of every row, so its share of dw stays in registers for the whole kernel (one global
// reduction per column and block at the end, no shared-memory atomics), each row is read once, and the R rows
// of a group are loaded together (2 R VPT 16-byte loads in flight per thread).
template <int VPT, int R>
__global__ void __launch_bounds__(512) rmsnorm_bwd_cols_kernel(const __nv_bfloat16* __restrict__ dy,
                                                               const __nv_bfloat16* __restrict__ x,
                                                               const __nv_bfloat16* __restrict__ w,
                                                               const float* __restrict__ rstd,
                                                               const __nv_bfloat16* __restrict__ dres,
                                                               __nv_bfloat16* __restrict__ dx,
                                                               float* __restrict__ dw_accum, int rows, int H) {
  __shared__ float red[2][R][16];
  const int nvec = H >> 3;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float fw[VPT][8], dw[VPT][8];
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int i = threadIdx.x + 512 * k;
    uint4 wv = make_uint4(0, 0, 0, 0);
    if (i < nvec) wv = __ldg(reinterpret_cast<const uint4*>(w) + i);
    unpack8(wv, fw[k]);
#pragma unroll
    for (int j = 0; j < 8; ++j) dw[k][j] = 0.f;
  }
  int it = 0;
  for (int row0 = blockIdx.x * R; row0 < rows; row0 += gridDim.x * R, ++it) {
    uint4 xv[R][VPT], dv[R][VPT];
    float rs[R];
#pragma unroll
    for (int q = 0; q < R; ++q) {
      const int row = row0 + q;
      rs[q] = row < rows ? rstd[row] : 0.f;
#pragma unroll
      for (int k = 0; k < VPT; ++k) {
        const int i = threadIdx.x + 512 * k;
        const bool in = row < rows && i < nvec;
        xv[q][k] = in ? __ldcs(reinterpret_cast<const uint4*>(x + (size_t)row * H) + i) : make_uint4(0, 0, 0, 0);
        dv[q][k] = in ? __ldcs(reinterpret_cast<const uint4*>(dy + (size_t)row * H) + i) : make_uint4(0, 0, 0, 0);
      }
    }
    float dot[R];
#pragma unroll
    for (int q = 0; q < R; ++q) {
      float a = 0.f;
#pragma unroll
      for (int k = 0; k < VPT; ++k) {
        float fx[8], fd[8];
        unpack8(xv[q][k], fx);
        unpack8(dv[q][k], fd);
#pragma unroll
        for (int j = 0; j < 8; ++j) a += fd[j] * fw[k][j] * fx[j];
      }
      a = warp_sum(a);
      if (lane == 0) red[it & 1][q][warp] = a;
    }
    __syncthreads();   // red[] of this parity is next written two iterations later, behind the next barrier
#pragma unroll
    for (int q = 0; q < R; ++q) {
      float a = lane < 16 ? red[it & 1][q][lane] : 0.f;
      dot[q] = warp_sum(a) * rs[q] / (float)H;
    }
#pragma unroll
    for (int q = 0; q < R; ++q) {
      const int row = row0 + q;
#pragma unroll
      for (int k = 0; k < VPT; ++k) {
        const int i = threadIdx.x + 512 * k;
        if (row < rows && i < nvec) {
          float fx[8], fd[8], o[8];
          unpack8(xv[q][k], fx);
          unpack8(dv[q][k], fd);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float xh = fx[j] * rs[q];
            o[j] = rs[q] * (fd[j] * fw[k][j] - xh * dot[q]);
            dw[k][j] += fd[j] * xh;
          }
          if (dres != nullptr) {  // gradient arriving through the residual branch
            float fr[8];
            unpack8(__ldcs(reinterpret_cast<const uint4*>(dres + (size_t)row * H) + i), fr);
#pragma unroll
            for (int j = 0; j < 8; ++j) o[j] += fr[j];
          }
          reinterpret_cast<uint4*>(dx + (size_t)row * H)[i] = pack8(o);
        }
      }
    }
  }
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int i = threadIdx.x + 512 * k;
    if (i < nvec) {
#pragma unroll
      for (int j = 0; j < 8; ++j) atomicAdd(&dw_accum[i * 8 + j], dw[k][j]);
    }
  }
}

// ------------------------------------------------------------------------------------------
// RoPE (rotate-half pairing i <-> i + D/2) applied to the Q and K column blocks of a fused
// [tokens, (Hq + 2 Hkv) * D] projection. cos/sin come from a per-token table [tokens, D/2] so
// any position layout (zigzag context-parallel chunks included) is a table lookup.
// K (rotated) and V can be written to separate [tokens, Hkv, D] buffers, e.g. peer-visible ones.
// sign = +1 forward, -1 backward (inverse rotation of the gradients).
// ------------------------------------------------------------------------------------------
__global__ void rope_qkv_kernel(__nv_bfloat16* __restrict__ qkv, const float* __restrict__ cos_t,
                                const float* __restrict__ sin_t, __nv_bfloat16* __restrict__ k_out,
                                __nv_bfloat16* __restrict__ v_out, int tokens, int tokens_per_seq, int Hq, int Hkv,
                                int D, float sign) {
  // one thread handles 8 consecutive pair indices (i .. i+7) of one head of one token
  const int half = D >> 1;
  const int vec_per_head = half >> 3;
  const int heads = Hq + Hkv + (v_out != nullptr ? Hkv : 0);
  const size_t total = (size_t)tokens * heads * vec_per_head;
  const int row_stride = (Hq + 2 * Hkv) * D;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const int v = (int)(idx % vec_per_head);
    const int h = (int)((idx / vec_per_head) % heads);
    const int t = (int)(idx / ((size_t)vec_per_head * heads));
    __nv_bfloat16* src = qkv + (size_t)t * row_stride + (size_t)h * D + v * 8;
    if (h >= Hq + Hkv) {
      // V head: plain copy of both halves into v_out
      __nv_bfloat16* dst = v_out + ((size_t)t * Hkv + (h - Hq - Hkv)) * D + v * 8;
      *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(src);
      *reinterpret_cast<uint4*>(dst + half) = *reinterpret_cast<const uint4*>(src + half);
      continue;
    }
    const int tp = t % tokens_per_seq;
    float lo[8], hi[8], c[8], s[8], olo[8], ohi[8];
    unpack8(*reinterpret_cast<const uint4*>(src), lo);
    unpack8(*reinterpret_cast<const uint4*>(src + half), hi);
    const float4* cp = reinterpret_cast<const float4*>(cos_t + (size_t)tp * half + v * 8);
    const float4* sp = reinterpret_cast<const float4*>(sin_t + (size_t)tp * half + v * 8);
    float4 c0 = cp[0], c1 = cp[1], s0 = sp[0], s1 = sp[1];
    c[0] = c0.x; c[1] = c0.y; c[2] = c0.z; c[3] = c0.w; c[4] = c1.x; c[5] = c1.y; c[6] = c1.z; c[7] = c1.w;
    s[0] = s0.x; s[1] = s0.y; s[2] = s0.z; s[3] = s0.w; s[4] = s1.x; s[5] = s1.y; s[6] = s1.z; s[7] = s1.w;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float sj = s[j] * sign;
      olo[j] = lo[j] * c[j] - hi[j] * sj;
      ohi[j] = hi[j] * c[j] + lo[j] * sj;
    }
    __nv_bfloat16* dst = src;
    if (h >= Hq && k_out != nullptr) dst = k_out + ((size_t)t * Hkv + (h - Hq)) * D + v * 8;
    *reinterpret_cast<uint4*>(dst) = pack8(olo);
    *reinterpret_cast<uint4*>(dst + half) = pack8(ohi);
  }
}

// Backward of the QKV split: fp32 dQ [tokens,Hq,D], dK, dV [tokens,Hkv,D] -> bf16 d(qkv)
// [tokens, (Hq+2Hkv)*D], applying the inverse rotation to the Q and K parts.
__global__ void rope_bwd_pack_kernel(const float* __restrict__ dq, const float* __restrict__ dk,
                                     const float* __restrict__ dv, const float* __restrict__ cos_t,
                                     const float* __restrict__ sin_t, __nv_bfloat16* __restrict__ dqkv, int tokens,
                                     int tokens_per_seq, int Hq, int Hkv, int D) {
  const int half = D >> 1;
  const int vec_per_head = half >> 3;
  const int heads = Hq + 2 * Hkv;
  const size_t total = (size_t)tokens * heads * vec_per_head;
  const int row_stride = heads * D;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const int v = (int)(idx % vec_per_head);
    const int h = (int)((idx / vec_per_head) % heads);
    const int t = (int)(idx / ((size_t)vec_per_head * heads));
    const float* src;
    if (h < Hq) src = dq + ((size_t)t * Hq + h) * D;
    else if (h < Hq + Hkv) src = dk + ((size_t)t * Hkv + (h - Hq)) * D;
    else src = dv + ((size_t)t * Hkv + (h - Hq - Hkv)) * D;
    src += v * 8;
    float lo[8], hi[8], olo[8], ohi[8];
    {
      const float4 a = reinterpret_cast<const float4*>(src)[0], b = reinterpret_cast<const float4*>(src)[1];
      const float4 c = reinterpret_cast<const float4*>(src + half)[0], d = reinterpret_cast<const float4*>(src + half)[1];
      lo[0] = a.x; lo[1] = a.y; lo[2] = a.z; lo[3] = a.w; lo[4] = b.x; lo[5] = b.y; lo[6] = b.z; lo[7] = b.w;
      hi[0] = c.x; hi[1] = c.y; hi[2] = c.z; hi[3] = c.w; hi[4] = d.x; hi[5] = d.y; hi[6] = d.z; hi[7] = d.w;
    }
    if (h < Hq + Hkv) {
      const int tp = t % tokens_per_seq;
      const float* cp = cos_t + (size_t)tp * half + v * 8;
      const float* sp = sin_t + (size_t)tp * half + v * 8;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float c = cp[j], sj = -sp[j];
        olo[j] = lo[j] * c - hi[j] * sj;
        ohi[j] = hi[j] * c + lo[j] * sj;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) { olo[j] = lo[j]; ohi[j] = hi[j]; }
    }
    __nv_bfloat16* dst = dqkv + (size_t)t * row_stride + (size_t)h * D + v * 8;
    *reinterpret_cast<uint4*>(dst) = pack8(olo);
    *reinterpret_cast<uint4*>(dst + half) = pack8(ohi);
  }
}

// ------------------------------------------------------------------------------------------
// SwiGLU on a fused [tokens, 2F] gate|up projection.
// ------------------------------------------------------------------------------------------
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ h, size_t tokens,
                                  int F) {
  const int vec_per_row = F >> 3;
  const size_t total = tokens * vec_per_row;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / vec_per_row;
    const int v = (int)(idx % vec_per_row);
    const __nv_bfloat16* row = gu + t * (size_t)(2 * F);
    float g[8], u[8], o[8];
    unpack8(*reinterpret_cast<const uint4*>(row + v * 8), g);
    unpack8(*reinterpret_cast<const uint4*>(row + F + v * 8), u);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = g[j] / (1.f + __expf(-g[j])) * u[j];
    *reinterpret_cast<uint4*>(h + t * (size_t)F + v * 8) = pack8(o);
  }
}

__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ gu, const __nv_bfloat16* __restrict__ dh,
                                  __nv_bfloat16* __restrict__ dgu, size_t tokens, int F) {
  const int vec_per_row = F >> 3;
  const size_t total = tokens * vec_per_row;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / vec_per_row;
    const int v = (int)(idx % vec_per_row);
    const __nv_bfloat16* row = gu + t * (size_t)(2 * F);
    float g[8], u[8], d[8], dg[8], du[8];
    unpack8(*reinterpret_cast<const uint4*>(row + v * 8), g);
    unpack8(*reinterpret_cast<const uint4*>(row + F + v * 8), u);
    unpack8(*reinterpret_cast<const uint4*>(dh + t * (size_t)F + v * 8), d);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float sg = 1.f / (1.f + __expf(-g[j]));
      const float silu = g[j] * sg;
      du[j] = d[j] * silu;
      dg[j] = d[j] * u[j] * (sg + silu * (1.f - sg));
    }
    __nv_bfloat16* orow = dgu + t * (size_t)(2 * F);
    *reinterpret_cast<uint4*>(orow + v * 8) = pack8(dg);
    *reinterpret_cast<uint4*>(orow + F + v * 8) = pack8(du);
  }
}

// ------------------------------------------------------------------------------------------
// Embedding gather and its fp32 scatter-add gradient.
// ------------------------------------------------------------------------------------------
__global__ void embedding_fwd_kernel(const int64_t* __restrict__ ids, const __nv_bfloat16* __restrict__ table,
                                     __nv_bfloat16* __restrict__ out, size_t tokens, int H, int vocab) {
  const int vec_per_row = H >> 3;
  const size_t total = tokens * vec_per_row;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / vec_per_row;
    const int v = (int)(idx % vec_per_row);
    int64_t id = ids[t];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
    reinterpret_cast<uint4*>(out + t * (size_t)H)[v] = reinterpret_cast<const uint4*>(table + (size_t)id * H)[v];
  }
}
__global__ void embedding_bwd_kernel(const int64_t* __restrict__ ids, const __nv_bfloat16* __restrict__ dout,
                                     float* __restrict__ dtable, size_t tokens, int H, int vocab) {
  const int vec_per_row = H >> 3;
  const size_t total = tokens * vec_per_row;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / vec_per_row;
    const int v = (int)(idx % vec_per_row);
    int64_t id = ids[t];
    if (id < 0 || id >= vocab) continue;
    float f[8];
    unpack8(reinterpret_cast<const uint4*>(dout + t * (size_t)H)[v], f);
    float* dst = dtable + (size_t)id * H + v * 8;
#pragma unroll
    for (int j = 0; j < 8; ++j) atomicAdd(dst + j, f[j]);
  }
}

// ------------------------------------------------------------------------------------------
// Softmax cross-entropy over one chunk of logits, forward and backward in one kernel: the logits
// are overwritten by (softmax - onehot) * grad_scale, the per-token loss goes to loss[row].
// One block per row; an online (max, sum) pass and a write pass.
// ------------------------------------------------------------------------------------------
__global__ void ce_fwd_bwd_kernel(__nv_bfloat16* __restrict__ logits, const int64_t* __restrict__ targets,
                                  float* __restrict__ loss, int V, int ld, float grad_scale, int ignore_index) {
  __shared__ float s_m[32], s_l[32];
  const int row = blockIdx.x;
  __nv_bfloat16* lr = logits + (size_t)row * ld;
  const int nvec = V >> 3;
  float m = -1.0e30f, l = 0.f;  // finite sentinel: idle threads must not produce inf - inf
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
    float f[8];
    unpack8(reinterpret_cast<const uint4*>(lr)[i], f);
    float cm = f[0];
#pragma unroll
    for (int j = 1; j < 8; ++j) cm = fmaxf(cm, f[j]);
    const float nm = fmaxf(m, cm);
    float acc = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) acc += __expf(f[j] - nm);
    l = l * __expf(m - nm) + acc;
    m = nm;
  }
  // block reduction of (m, l)
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  float wm = warp_max(m);
  float wl = warp_sum(l * __expf(m - wm));
  if (lane == 0) { s_m[warp] = wm; s_l[warp] = wl; }
  __syncthreads();
  float bm = lane < nwarps ? s_m[lane] : -1.0e30f;
  float bl = lane < nwarps ? s_l[lane] : 0.f;
  const float gm = warp_max(bm);
  const float gl = warp_sum(bl * __expf(bm - gm));
  const int64_t tgt = targets[row];
  const bool ignored = (tgt == ignore_index) || tgt < 0 || tgt >= V;
  const float lse = gm + __logf(gl);
  if (threadIdx.x == 0) loss[row] = ignored ? 0.f : lse - __bfloat162float(lr[tgt]);
  __syncthreads();
  const float inv = 1.f / gl;
  const float gs = ignored ? 0.f : grad_scale;
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
    float f[8];
    unpack8(reinterpret_cast<const uint4*>(lr)[i], f);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float pj = __expf(f[j] - gm) * inv;
      if ((int64_t)(i * 8 + j) == tgt) pj -= 1.f;
      f[j] = pj * gs;
    }
    reinterpret_cast<uint4*>(lr)[i] = pack8(f);
  }
}

// ------------------------------------------------------------------------------------------
// e4m3 quantisation of K or V: x [tokens, Hkv, D] -> q (e4m3) + one fp32 scale per (128-token
// block, head): scale = absmax / 448. One block (256 threads) per (token block, head).
// ------------------------------------------------------------------------------------------
__global__ void kv_quant_e4m3_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ q,
                                     float* __restrict__ scales, float* __restrict__ scales_pow2, int tokens, int Hkv,
                                     int D, int block_tokens) {
  __shared__ float s_red[8];
  __shared__ float s_scale;
  const int blk = blockIdx.x / Hkv, head = blockIdx.x % Hkv;
  const int t0 = blk * block_tokens;
  const int vec_per_tok = D >> 3;
  const int nvec = block_tokens * vec_per_tok;
  float amax = 0.f;
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
    const int t = t0 + i / vec_per_tok;
    if (t >= tokens) break;
    float f[8];
    unpack8(reinterpret_cast<const uint4*>(x + ((size_t)t * Hkv + head) * D)[i % vec_per_tok], f);
#pragma unroll
    for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(f[j]));
  }
  amax = warp_max(amax);
  if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = amax;
  __syncthreads();
  if (threadIdx.x == 0) {
    float a = 0.f;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) a = fmaxf(a, s_red[w]);
    float sc = a > 0.f ? a / 448.f : 1.f;
    s_scale = sc;
    scales[(size_t)blk * Hkv + head] = sc;
    if (scales_pow2 != nullptr) scales_pow2[(size_t)blk * Hkv + head] = exp2f(ceilf(log2f(sc)));
  }
  __syncthreads();
  const float inv = 1.f / s_scale;
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
    const int t = t0 + i / vec_per_tok;
    if (t >= tokens) break;
    float f[8];
    const size_t off = ((size_t)t * Hkv + head) * D + (size_t)(i % vec_per_tok) * 8;
    unpack8(*reinterpret_cast<const uint4*>(x + off), f);
    uint32_t lo = 0, hi = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      lo |= (uint32_t)__nv_cvt_float_to_fp8(f[j] * inv, __NV_SATFINITE, __NV_E4M3) << (8 * j);
      hi |= (uint32_t)__nv_cvt_float_to_fp8(f[4 + j] * inv, __NV_SATFINITE, __NV_E4M3) << (8 * j);
    }
    *reinterpret_cast<uint2*>(q + off) = make_uint2(lo, hi);
  }
}

__global__ void kv_dequant_e4m3_kernel(const uint8_t* __restrict__ q, const float* __restrict__ scales,
                                       __nv_bfloat16* __restrict__ x, size_t tokens, int Hkv, int D, int block_tokens) {
  const int vec_per_tok = D >> 3;
  const size_t total = tokens * Hkv * vec_per_tok;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const size_t th = idx / vec_per_tok;  // token * Hkv + head
    const size_t t = th / Hkv;
    const int head = (int)(th % Hkv);
    const float sc = scales[(t / block_tokens) * Hkv + head];
    const uint2 u = *reinterpret_cast<const uint2*>(q + idx * 8);
    float f[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      __half_raw h0 = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)((u.x >> (8 * j)) & 0xff), __NV_E4M3);
      __half_raw h1 = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)((u.y >> (8 * j)) & 0xff), __NV_E4M3);
      f[j] = __half2float(__half(h0)) * sc;
      f[4 + j] = __half2float(__half(h1)) * sc;
    }
    *reinterpret_cast<uint4*>(x + idx * 8) = pack8(f);
  }
}

// ------------------------------------------------------------------------------------------
// AdamW on a flat shard. The fp32 master weight is kept as two 16-bit halves: `p_hi` is the bf16
// parameter the GEMMs read (round-half-up of the master) and `p_lo` the signed remainder, so the
// pair reconstructs the fp32 value exactly at 4 bytes per parameter.
// grad_scale_ptr (optional) holds one fp32 factor computed on the device (e.g. 1/accum * clip).
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ float join_master(uint16_t hi, int16_t lo) {
  const uint32_t bits = ((uint32_t)hi << 16) + (uint32_t)(int32_t)lo;
  return __uint_as_float(bits);
}
__device__ __forceinline__ void split_master(float w, uint16_t& hi, int16_t& lo) {
  const uint32_t bits = __float_as_uint(w);
  const uint32_t h = (bits + 0x8000u) >> 16;
  hi = (uint16_t)h;
  lo = (int16_t)(int32_t)(bits - (h << 16));
}

__global__ void adamw_kernel(uint16_t* __restrict__ p_hi, int16_t* __restrict__ p_lo, float* __restrict__ m,
                             float* __restrict__ v, const float* __restrict__ g, size_t n, float lr, float beta1,
                             float beta2, float eps, float weight_decay, float bias1, float bias2, float grad_scale,
                             const float* __restrict__ grad_scale_ptr) {
  const float gs = grad_scale * (grad_scale_ptr != nullptr ? *grad_scale_ptr : 1.f);
  const size_t nvec = n >> 2;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (size_t)gridDim.x * blockDim.x) {
    const float4 gg = reinterpret_cast<const float4*>(g)[i];
    float4 mm = reinterpret_cast<float4*>(m)[i];
    float4 vv = reinterpret_cast<float4*>(v)[i];
    const uint2 hi = reinterpret_cast<uint2*>(p_hi)[i];
    const uint2 lo = reinterpret_cast<uint2*>(p_lo)[i];
    const uint16_t h[4] = {(uint16_t)(hi.x & 0xffff), (uint16_t)(hi.x >> 16), (uint16_t)(hi.y & 0xffff), (uint16_t)(hi.y >> 16)};
    const int16_t l[4] = {(int16_t)(lo.x & 0xffff), (int16_t)(lo.x >> 16), (int16_t)(lo.y & 0xffff), (int16_t)(lo.y >> 16)};
    float gr[4] = {gg.x * gs, gg.y * gs, gg.z * gs, gg.w * gs};
    float ma[4] = {mm.x, mm.y, mm.z, mm.w};
    float va[4] = {vv.x, vv.y, vv.z, vv.w};
    uint16_t nh[4];
    int16_t nl[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float w = join_master(h[j], l[j]);
      ma[j] = beta1 * ma[j] + (1.f - beta1) * gr[j];
      va[j] = beta2 * va[j] + (1.f - beta2) * gr[j] * gr[j];
      const float mhat = ma[j] / bias1;
      const float vhat = va[j] / bias2;
      w = w * (1.f - lr * weight_decay) - lr * mhat / (sqrtf(vhat) + eps);
      split_master(w, nh[j], nl[j]);
    }
    reinterpret_cast<float4*>(m)[i] = make_float4(ma[0], ma[1], ma[2], ma[3]);
    reinterpret_cast<float4*>(v)[i] = make_float4(va[0], va[1], va[2], va[3]);
    reinterpret_cast<uint2*>(p_hi)[i] = make_uint2((uint32_t)nh[0] | ((uint32_t)nh[1] << 16), (uint32_t)nh[2] | ((uint32_t)nh[3] << 16));
    reinterpret_cast<uint2*>(p_lo)[i] =
        make_uint2((uint32_t)(uint16_t)nl[0] | ((uint32_t)(uint16_t)nl[1] << 16), (uint32_t)(uint16_t)nl[2] | ((uint32_t)(uint16_t)nl[3] << 16));
  }
}

// out[i] = sum over r of slots[r * n + i]: second half of the fused reduce-scatter (the GEMM epilogues of
// every rank stored their bf16 partial rows into this rank's slots); fp32 sum, one rounding.
__global__ void sum_slots_bf16_kernel(const __nv_bfloat16* __restrict__ slots, int ranks, size_t n,
                                      __nv_bfloat16* __restrict__ out) {
  const size_t nvec = n >> 3;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (size_t)gridDim.x * blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int r = 0; r < ranks; ++r) {
      const uint4 v = reinterpret_cast<const uint4*>(slots + (size_t)r * n)[i];
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        acc[2 * j] += __uint_as_float(w[j] << 16);
        acc[2 * j + 1] += __uint_as_float(w[j] & 0xffff0000u);
      }
    }
    uint4 o;
    uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const __nv_bfloat162 h = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
      ow[j] = *reinterpret_cast<const uint32_t*>(&h);
    }
    reinterpret_cast<uint4*>(out)[i] = o;
  }
}

// sum of squares of a flat fp32 buffer, accumulated into out[0] (caller zeroes it)
__global__ void sumsq_kernel(const float* __restrict__ g, size_t n, float* __restrict__ out) {
  __shared__ float s[32];
  float acc = 0.f;
  const size_t nvec = n >> 2;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (size_t)gridDim.x * blockDim.x) {
    const float4 a = reinterpret_cast<const float4*>(g)[i];
    acc += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
  }
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) s[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < (blockDim.x >> 5) ? s[threadIdx.x] : 0.f;
    t = warp_sum(t);
    if (threadIdx.x == 0) atomicAdd(out, t);
  }
}

// clip coefficient from the accumulated sum of squares: coef = min(1, max_norm / (sqrt(ss)*scale + 1e-6))
__global__ void clip_coef_kernel(const float* __restrict__ sumsq, float scale, float max_norm, float* __restrict__ coef,
                                 float* __restrict__ norm_out) {
  const float norm = sqrtf(*sumsq) * scale;
  if (norm_out != nullptr) *norm_out = norm;
  *coef = max_norm > 0.f ? fminf(1.f, max_norm / (norm + 1e-6f)) : 1.f;
}

inline int grid_for(size_t work_items, int threads, int sm_count) {
  size_t blocks = (work_items + threads - 1) / threads;
  size_t cap = (size_t)sm_count * 16;
  return (int)(blocks < cap ? (blocks == 0 ? 1 : blocks) : cap);
}

}  // namespace

void launch_rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd, int rows, int H, float eps,
                        cudaStream_t st) {
  if (rows == 0) return;
  const int wpb = 4;
  const unsigned grid = (rows + wpb - 1) / wpb;
  auto xb = (const __nv_bfloat16*)x;
  auto wb = (const __nv_bfloat16*)w;
  auto yb = (__nv_bfloat16*)y;
  switch (H) {
    case 2048: rmsnorm_fwd_regs_kernel<8><<<grid, wpb * 32, 0, st>>>(xb, wb, yb, rstd, rows, eps); break;
    case 4096: rmsnorm_fwd_regs_kernel<16><<<grid, wpb * 32, 0, st>>>(xb, wb, yb, rstd, rows, eps); break;
    default: rmsnorm_fwd_kernel<<<grid, wpb * 32, 0, st>>>(xb, wb, yb, rstd, rows, H, eps);
  }
}
void launch_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, const void* dres, void* dx,
                        float* dw_accum, int rows, int H, int sm_count, cudaStream_t st) {
  if (rows == 0) return;
  auto dyb = (const __nv_bfloat16*)dy;
  auto xb = (const __nv_bfloat16*)x;
  auto wb = (const __nv_bfloat16*)w;
  auto rb = (const __nv_bfloat16*)dres;
  auto dxb = (__nv_bfloat16*)dx;
  const int nvec = H / 8;
  if (nvec <= 1024) {
    // one resident block of 512 threads per SM (the row group lives in registers): a persistent grid
    const int R = nvec <= 512 ? 4 : 2;
    int grid = sm_count;
    const int max_grid = (rows + R - 1) / R;
    if (grid > max_grid) grid = max_grid;
    if (nvec <= 512)
      rmsnorm_bwd_cols_kernel<1, 4><<<grid, 512, 0, st>>>(dyb, xb, wb, rstd, rb, dxb, dw_accum, rows, H);
    else
      rmsnorm_bwd_cols_kernel<2, 2><<<grid, 512, 0, st>>>(dyb, xb, wb, rstd, rb, dxb, dw_accum, rows, H);
    return;
  }
  const int threads = 256;
  int grid = sm_count * 4;
  const int max_grid = (rows + 7) / 8;
  if (grid > max_grid) grid = max_grid;
  rmsnorm_bwd_kernel<<<grid, threads, H * sizeof(float), st>>>(dyb, xb, wb, rstd, rb, dxb, dw_accum, rows, H);
}
void launch_rope_qkv(void* qkv, const float* cos_t, const float* sin_t, void* k_out, void* v_out, int tokens,
                     int tokens_per_seq, int Hq, int Hkv, int D, float sign, int sm_count, cudaStream_t st) {
  if (tokens == 0) return;
  const int heads = Hq + Hkv + (v_out != nullptr ? Hkv : 0);
  const size_t total = (size_t)tokens * heads * (D / 16);
  rope_qkv_kernel<<<grid_for(total, 256, sm_count), 256, 0, st>>>((__nv_bfloat16*)qkv, cos_t, sin_t,
                                                                  (__nv_bfloat16*)k_out, (__nv_bfloat16*)v_out, tokens,
                                                                  tokens_per_seq, Hq, Hkv, D, sign);
}
void launch_rope_bwd_pack(const float* dq, const float* dk, const float* dv, const float* cos_t, const float* sin_t,
                          void* dqkv, int tokens, int tokens_per_seq, int Hq, int Hkv, int D, int sm_count,
                          cudaStream_t st) {
  if (tokens == 0) return;
  const size_t total = (size_t)tokens * (Hq + 2 * Hkv) * (D / 16);
  rope_bwd_pack_kernel<<<grid_for(total, 256, sm_count), 256, 0, st>>>(dq, dk, dv, cos_t, sin_t, (__nv_bfloat16*)dqkv,
                                                                       tokens, tokens_per_seq, Hq, Hkv, D);
}
void launch_swiglu_fwd(const void* gu, void* h, size_t tokens, int F, int sm_count, cudaStream_t st) {
  if (tokens == 0) return;
  swiglu_fwd_kernel<<<grid_for(tokens * (F / 8), 256, sm_count), 256, 0, st>>>((const __nv_bfloat16*)gu,
                                                                               (__nv_bfloat16*)h, tokens, F);
}
void launch_swiglu_bwd(const void* gu, const void* dh, void* dgu, size_t tokens, int F, int sm_count,
                       cudaStream_t st) {
  if (tokens == 0) return;
  swiglu_bwd_kernel<<<grid_for(tokens * (F / 8), 256, sm_count), 256, 0, st>>>(
      (const __nv_bfloat16*)gu, (const __nv_bfloat16*)dh, (__nv_bfloat16*)dgu, tokens, F);
}
void launch_embedding_fwd(const int64_t* ids, const void* table, void* out, size_t tokens, int H, int vocab,
                          int sm_count, cudaStream_t st) {
  if (tokens == 0) return;
  embedding_fwd_kernel<<<grid_for(tokens * (H / 8), 256, sm_count), 256, 0, st>>>(ids, (const __nv_bfloat16*)table,
                                                                                  (__nv_bfloat16*)out, tokens, H, vocab);
}
void launch_embedding_bwd(const int64_t* ids, const void* dout, float* dtable, size_t tokens, int H, int vocab,
                          int sm_count, cudaStream_t st) {
  if (tokens == 0) return;
  embedding_bwd_kernel<<<grid_for(tokens * (H / 8), 256, sm_count), 256, 0, st>>>(ids, (const __nv_bfloat16*)dout,
                                                                                  dtable, tokens, H, vocab);
}
void launch_ce_fwd_bwd(void* logits, const int64_t* targets, float* loss, int rows, int V, int ld, float grad_scale,
                       int ignore_index, cudaStream_t st) {
  if (rows == 0) return;
  ce_fwd_bwd_kernel<<<rows, 512, 0, st>>>((__nv_bfloat16*)logits, targets, loss, V, ld, grad_scale, ignore_index);
}
void launch_kv_quant_e4m3(const void* x, void* q, float* scales, float* scales_pow2, int tokens, int Hkv, int D,
                          int block_tokens, cudaStream_t st) {
  if (tokens == 0) return;
  const int blocks = (tokens + block_tokens - 1) / block_tokens;
  kv_quant_e4m3_kernel<<<blocks * Hkv, 256, 0, st>>>((const __nv_bfloat16*)x, (uint8_t*)q, scales, scales_pow2, tokens,
                                                     Hkv, D, block_tokens);
}
void launch_kv_dequant_e4m3(const void* q, const float* scales, void* x, size_t tokens, int Hkv, int D,
                            int block_tokens, int sm_count, cudaStream_t st) {
  if (tokens == 0) return;
  kv_dequant_e4m3_kernel<<<grid_for(tokens * Hkv * (D / 8), 256, sm_count), 256, 0, st>>>(
      (const uint8_t*)q, scales, (__nv_bfloat16*)x, tokens, Hkv, D, block_tokens);
}
void launch_adamw(void* p_hi, void* p_lo, float* m, float* v, const float* g, size_t n, float lr, float beta1,
                  float beta2, float eps, float weight_decay, int step, float grad_scale, const float* grad_scale_ptr,
                  int sm_count, cudaStream_t st) {
  if (n == 0) return;
  const float bias1 = 1.f - powf(beta1, (float)step);
  const float bias2 = 1.f - powf(beta2, (float)step);
  adamw_kernel<<<grid_for(n / 4, 256, sm_count), 256, 0, st>>>((uint16_t*)p_hi, (int16_t*)p_lo, m, v, g, n, lr, beta1,
                                                               beta2, eps, weight_decay, bias1, bias2, grad_scale,
                                                               grad_scale_ptr);
}
void launch_sum_slots_bf16(const void* slots, int ranks, size_t n, void* out, int sm_count, cudaStream_t st) {
  if (n == 0) return;
  sum_slots_bf16_kernel<<<grid_for(n / 8, 256, sm_count), 256, 0, st>>>((const __nv_bfloat16*)slots, ranks, n,
                                                                         (__nv_bfloat16*)out);
}
void launch_sumsq(const float* g, size_t n, float* out, int sm_count, cudaStream_t st) {
  if (n == 0) return;
  sumsq_kernel<<<grid_for(n / 4, 256, sm_count), 256, 0, st>>>(g, n, out);
}
void launch_clip_coef(const float* sumsq, float scale, float max_norm, float* coef, float* norm_out, cudaStream_t st) {
  clip_coef_kernel<<<1, 1, 0, st>>>(sumsq, scale, max_norm, coef, norm_out);
}

}  // namespace zx
