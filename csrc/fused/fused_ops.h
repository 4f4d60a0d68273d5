// Launchers of the bandwidth-bound kernels (raw pointers + stream; bf16 data unless noted).
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace zx {

void launch_rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd, int rows, int H, float eps,
                        cudaStream_t st);
void launch_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, const void* dres, void* dx,
                        float* dw_accum, int rows, int H, int sm_count, cudaStream_t st);
void launch_rope_bwd_pack(const float* dq, const float* dk, const float* dv, const float* cos_t, const float* sin_t,
                          void* dqkv, int tokens, int tokens_per_seq, int Hq, int Hkv, int D, int sm_count,
                          cudaStream_t st);
void launch_rope_qkv(void* qkv, const float* cos_t, const float* sin_t, void* k_out, void* v_out, int tokens,
                     int tokens_per_seq, int Hq, int Hkv, int D, float sign, int sm_count, cudaStream_t st);
void launch_swiglu_fwd(const void* gu, void* h, size_t tokens, int F, int sm_count, cudaStream_t st);
void launch_swiglu_bwd(const void* gu, const void* dh, void* dgu, size_t tokens, int F, int sm_count, cudaStream_t st);
void launch_embedding_fwd(const int64_t* ids, const void* table, void* out, size_t tokens, int H, int vocab,
                          int sm_count, cudaStream_t st);
void launch_embedding_bwd(const int64_t* ids, const void* dout, float* dtable, size_t tokens, int H, int vocab,
                          int sm_count, cudaStream_t st);
void launch_ce_fwd_bwd(void* logits, const int64_t* targets, float* loss, int rows, int V, int ld, float grad_scale,
                       int ignore_index, cudaStream_t st);
void launch_kv_quant_e4m3(const void* x, void* q, float* scales, float* scales_pow2, int tokens, int Hkv, int D,
                          int block_tokens, cudaStream_t st);
void launch_kv_dequant_e4m3(const void* q, const float* scales, void* x, size_t tokens, int Hkv, int D,
                            int block_tokens, int sm_count, cudaStream_t st);
void launch_adamw(void* p_hi, void* p_lo, float* m, float* v, const float* g, size_t n, float lr, float beta1,
                  float beta2, float eps, float weight_decay, int step, float grad_scale, const float* grad_scale_ptr,
                  int sm_count, cudaStream_t st);
// out[i] = sum_r slots[r * n + i] (bf16 in, fp32 sum, bf16 out); n a multiple of 8
void launch_sum_slots_bf16(const void* slots, int ranks, size_t n, void* out, int sm_count, cudaStream_t st);
void launch_sumsq(const float* g, size_t n, float* out, int sm_count, cudaStream_t st);
void launch_clip_coef(const float* sumsq, float scale, float max_norm, float* coef, float* norm_out, cudaStream_t st);

}  // namespace zx
