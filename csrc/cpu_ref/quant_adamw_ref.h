// Scalar host restatements of two device kernels, used as oracles by the tests:
//  * the e4m3 K/V quantiser (csrc/fused/fused_ops.cu: one fp32 scale = absmax / 448 per (token block, head),
//    round to nearest even, saturate at +-448);
//  * one AdamW step on the split fp32 master (csrc/optim/zero_adamw.cu: master = bf16 high half + int16
//    remainder, round-half-up split, decoupled weight decay).
// The reference project has no native code, hence no counterpart.
#pragma once
#include <cstddef>
#include <cstdint>

namespace zx {

// x [tokens, heads, dim] fp32 -> q (e4m3 codes) and scales [ceil(tokens / block_tokens), heads].
void quant_e4m3_ref(const float* x, uint8_t* q, float* scales, int64_t tokens, int heads, int dim, int block_tokens);
float e4m3_to_float(uint8_t code);
uint8_t float_to_e4m3_satfinite(float v);

// In place on n elements: p_hi (bf16 bits), p_lo (int16 remainder), m, v; g is the already scaled gradient.
void adamw_split_master_ref(uint16_t* p_hi, int16_t* p_lo, float* m, float* v, const float* g, size_t n, size_t decay_end,
                            float lr, float beta1, float beta2, float eps, float weight_decay, int step);

}  // namespace zx
