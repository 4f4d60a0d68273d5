#include "quant_adamw_ref.h"

#include <algorithm>
#include <cmath>
#include <cstring>

namespace zx {

float e4m3_to_float(uint8_t code) {
  const int sign = code >> 7, exp = (code >> 3) & 0xF, man = code & 7;
  float v;
  if (exp == 0) v = std::ldexp((float)man, -9);                 // subnormal: man * 2^-3 * 2^-6
  else if (exp == 15 && man == 7) v = NAN;                      // the only NaN encoding of e4m3 (no infinities)
  else v = std::ldexp(1.f + man / 8.f, exp - 7);
  return sign ? -v : v;
}

uint8_t float_to_e4m3_satfinite(float x) {
  if (std::isnan(x)) return 0x7F;
  const uint8_t sign = std::signbit(x) ? 0x80 : 0;
  float a = std::fabs(x);
  if (a >= 448.f) return sign | 0x7E;                           // saturate to the largest finite value
  if (a < std::ldexp(1.f, -10)) return sign;                    // below half of the smallest subnormal: zero
  int e;
  std::frexp(a, &e);                                            // a = f * 2^e, f in [0.5, 1)
  int exp = e - 1;                                              // a = (1.xxx) * 2^exp
  if (exp < -6) exp = -6;                                       // subnormal range shares the exponent -6
  const float step = std::ldexp(1.f, exp - 3);                  // spacing of representable values around a
  float qv = std::nearbyint(a / step) * step;                   // round to nearest even (default rounding mode)
  if (qv >= 448.f + 16.f) qv = 448.f;
  // encode qv
  if (qv < std::ldexp(1.f, -6)) return sign | (uint8_t)std::lround(qv / std::ldexp(1.f, -9));
  std::frexp(qv, &e);
  exp = e - 1;
  const int man = (int)std::lround((qv / std::ldexp(1.f, exp) - 1.f) * 8.f);
  return sign | (uint8_t)(((exp + 7) << 3) | man);
}

void quant_e4m3_ref(const float* x, uint8_t* q, float* scales, int64_t tokens, int heads, int dim, int block_tokens) {
  const int64_t n_blocks = (tokens + block_tokens - 1) / block_tokens;
  for (int64_t b = 0; b < n_blocks; ++b) {
    const int64_t t0 = b * block_tokens, t1 = std::min<int64_t>(tokens, t0 + block_tokens);
    for (int h = 0; h < heads; ++h) {
      float amax = 0.f;
      for (int64_t t = t0; t < t1; ++t)
        for (int d = 0; d < dim; ++d) amax = std::max(amax, std::fabs(x[(t * heads + h) * dim + d]));
      const float sc = amax > 0.f ? amax / 448.f : 1.f;
      scales[b * heads + h] = sc;
      const float inv = 1.f / sc;
      for (int64_t t = t0; t < t1; ++t)
        for (int d = 0; d < dim; ++d) {
          const int64_t i = (t * heads + h) * dim + d;
          q[i] = float_to_e4m3_satfinite(x[i] * inv);
        }
    }
  }
}

void adamw_split_master_ref(uint16_t* p_hi, int16_t* p_lo, float* m, float* v, const float* g, size_t n, size_t decay_end,
                            float lr, float beta1, float beta2, float eps, float weight_decay, int step) {
  const float bias1 = 1.f - std::pow(beta1, (float)step), bias2 = 1.f - std::pow(beta2, (float)step);
  for (size_t i = 0; i < n; ++i) {
    const uint32_t bits_in = ((uint32_t)p_hi[i] << 16) + (uint32_t)(int32_t)p_lo[i];
    float w;
    std::memcpy(&w, &bits_in, 4);
    m[i] = beta1 * m[i] + (1.f - beta1) * g[i];
    v[i] = beta2 * v[i] + (1.f - beta2) * g[i] * g[i];
    const float wd = i < decay_end ? weight_decay : 0.f;
    w = w * (1.f - lr * wd) - lr * (m[i] / bias1) / (std::sqrt(v[i] / bias2) + eps);
    uint32_t bits;
    std::memcpy(&bits, &w, 4);
    const uint32_t hh = (bits + 0x8000u) >> 16;
    p_hi[i] = (uint16_t)(hh & 0xffffu);
    p_lo[i] = (int16_t)((bits - (hh << 16)) & 0xffffu);
  }
}

}  // namespace zx
