// fp32 blockwise attention with an online softmax, OpenMP over (batch, head, query block).
// The reference names a ``flash_cpu.py`` among its deleted operators
// (ZENYX_2_0_DELIVERABLES.txt:195); no code of it exists.
#include "flash_cpu.h"

#include <algorithm>
#include <cmath>
#include <cstring>
#include <limits>

namespace zxh {

namespace {

constexpr int BLK = 64;

inline bool allowed(const CpuAttnShape& s, int64_t qp, int64_t kp) {
  if (s.causal && kp > qp) return false;
  if (s.window_blocks > 0) {
    const int64_t qb = qp / 128, kb = kp / 128;
    const int64_t dist = qb >= kb ? qb - kb : kb - qb;
    const bool in_window = dist < s.window_blocks;
    const bool is_global = s.global_every > 0 && (kb % s.global_every) == 0;
    if (!in_window && !is_global) return false;
  }
  return true;
}

}  // namespace

void flash_cpu_forward(const CpuAttnShape& s, const float* q, const float* k, const float* v, const int64_t* qpos,
                       const int64_t* kpos, float* o, float* lse, bool merge_prev) {
  const int G = s.Hq / s.Hkv;
  const int nqb = (s.Sq + BLK - 1) / BLK;
  const float NEG = -std::numeric_limits<float>::infinity();
#pragma omp parallel for collapse(3) schedule(dynamic)
  for (int b = 0; b < s.B; ++b)
    for (int h = 0; h < s.Hq; ++h)
      for (int qb = 0; qb < nqb; ++qb) {
        const int hk = h / G;
        const int q0 = qb * BLK, q1 = std::min(s.Sq, q0 + BLK);
        std::vector<float> acc((size_t)(q1 - q0) * s.D, 0.f), m(q1 - q0, NEG), l(q1 - q0, 0.f), sc(BLK);
        for (int k0 = 0; k0 < s.Skv; k0 += BLK) {
          const int k1 = std::min(s.Skv, k0 + BLK);
          for (int i = q0; i < q1; ++i) {
            const float* qi = q + (((size_t)b * s.Sq + i) * s.Hq + h) * s.D;
            float mx = NEG;
            for (int j = k0; j < k1; ++j) {
              float d = NEG;
              if (allowed(s, qpos[i], kpos[j])) {
                const float* kj = k + (((size_t)b * s.Skv + j) * s.Hkv + hk) * s.D;
                float dot = 0.f;
                for (int e = 0; e < s.D; ++e) dot += qi[e] * kj[e];
                d = dot * s.scale;
              }
              sc[j - k0] = d;
              mx = std::max(mx, d);
            }
            if (mx == NEG) continue;
            const int r = i - q0;
            const float m_new = std::max(m[r], mx);
            const float alpha = m[r] == NEG ? 0.f : std::exp(m[r] - m_new);
            float* a = acc.data() + (size_t)r * s.D;
            for (int e = 0; e < s.D; ++e) a[e] *= alpha;
            float sum = 0.f;
            for (int j = k0; j < k1; ++j) {
              if (sc[j - k0] == NEG) continue;
              const float p = std::exp(sc[j - k0] - m_new);
              sum += p;
              const float* vj = v + (((size_t)b * s.Skv + j) * s.Hkv + hk) * s.D;
              for (int e = 0; e < s.D; ++e) a[e] += p * vj[e];
            }
            l[r] = l[r] * alpha + sum;
            m[r] = m_new;
          }
        }
        for (int i = q0; i < q1; ++i) {
          const int r = i - q0;
          float* oi = o + (((size_t)b * s.Sq + i) * s.Hq + h) * s.D;
          float* li = lse + ((size_t)b * s.Hq + h) * s.Sq + i;
          const float lse_cur = l[r] > 0.f ? m[r] + std::log(l[r]) : NEG;
          const float inv = l[r] > 0.f ? 1.f / l[r] : 0.f;
          const float* a = acc.data() + (size_t)r * s.D;
          if (!merge_prev) {
            for (int e = 0; e < s.D; ++e) oi[e] = a[e] * inv;
            *li = lse_cur;
          } else {
            const float lp = *li;
            const float mx = std::max(lp, lse_cur);
            if (mx == NEG) continue;
            const float ep = lp == NEG ? 0.f : std::exp(lp - mx), ec = lse_cur == NEG ? 0.f : std::exp(lse_cur - mx);
            const float wp = ep / (ep + ec), wc = ec / (ep + ec) * inv;
            for (int e = 0; e < s.D; ++e) oi[e] = oi[e] * wp + a[e] * wc;
            *li = mx + std::log(ep + ec);
          }
        }
      }
}

void flash_cpu_backward(const CpuAttnShape& s, const float* q, const float* k, const float* v, const float* o,
                        const float* d_o, const float* lse, const int64_t* qpos, const int64_t* kpos, float* dq,
                        float* dk, float* dv) {
  const int G = s.Hq / s.Hkv;
  const float NEG = -std::numeric_limits<float>::infinity();
  std::memset(dq, 0, sizeof(float) * (size_t)s.B * s.Sq * s.Hq * s.D);
  // parallel over (batch, kv head): each thread owns its dK/dV rows, dq rows are private per q head
#pragma omp parallel for collapse(2) schedule(dynamic)
  for (int b = 0; b < s.B; ++b)
    for (int hk = 0; hk < s.Hkv; ++hk)
      for (int g = 0; g < G; ++g) {
        const int h = hk * G + g;
        for (int i = 0; i < s.Sq; ++i) {
          const float L = lse[((size_t)b * s.Hq + h) * s.Sq + i];
          if (L == NEG) continue;
          const size_t qoff = (((size_t)b * s.Sq + i) * s.Hq + h) * s.D;
          const float* qi = q + qoff;
          const float* doi = d_o + qoff;
          const float* oi = o + qoff;
          float delta = 0.f;
          for (int e = 0; e < s.D; ++e) delta += doi[e] * oi[e];
          float* dqi = dq + qoff;
          for (int j = 0; j < s.Skv; ++j) {
            if (!allowed(s, qpos[i], kpos[j])) continue;
            const size_t koff = (((size_t)b * s.Skv + j) * s.Hkv + hk) * s.D;
            const float* kj = k + koff;
            const float* vj = v + koff;
            float dot = 0.f, dp = 0.f;
            for (int e = 0; e < s.D; ++e) {
              dot += qi[e] * kj[e];
              dp += doi[e] * vj[e];
            }
            const float p = std::exp(dot * s.scale - L);
            const float ds = p * (dp - delta) * s.scale;
            float* dkj = dk + koff;
            float* dvj = dv + koff;
            for (int e = 0; e < s.D; ++e) {
              dqi[e] += ds * kj[e];
              dkj[e] += ds * qi[e];
              dvj[e] += p * doi[e];
            }
          }
        }
      }
}

}  // namespace zxh
