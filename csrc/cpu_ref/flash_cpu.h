// Blockwise (flash-style) attention on the CPU in fp32: the oracle for the GPU kernels and the
// timed CPU baseline. Same position-table masking as the GPU kernels.
#pragma once
#include <cstdint>
#include <vector>

namespace zxh {

struct CpuAttnShape {
  int B, Sq, Skv, Hq, Hkv, D;
  float scale;
  int causal, window_blocks, global_every;
};

// q [B,Sq,Hq,D], k/v [B,Skv,Hkv,D], qpos [Sq], kpos [Skv] (global token positions).
// o [B,Sq,Hq,D], lse [B,Hq,Sq]. With merge_prev the result is folded into the o/lse passed in.
void flash_cpu_forward(const CpuAttnShape& s, const float* q, const float* k, const float* v, const int64_t* qpos,
                       const int64_t* kpos, float* o, float* lse, bool merge_prev);

// dq [B,Sq,Hq,D] is overwritten; dk/dv [B,Skv,Hkv,D] are added to.
void flash_cpu_backward(const CpuAttnShape& s, const float* q, const float* k, const float* v, const float* o,
                        const float* d_o, const float* lse, const int64_t* qpos, const int64_t* kpos, float* dq,
                        float* dk, float* dv);

}  // namespace zxh
