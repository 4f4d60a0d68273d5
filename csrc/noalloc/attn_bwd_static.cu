// See attn_bwd_static.h. The scratch array and the code that takes its device address live in this
// one file: in host code the array's name is only a stand-in, so the address handed to the
// kernels comes from cudaGetSymbolAddress, looked up once per device with that device current.
#include "attn_bwd_static.h"

#include <cuda_runtime.h>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <exception>

#include "../attn/attn.h"

namespace {

static __device__ __align__(256) float g_delta_scratch[ZX_ATTN_BWD_NOALLOC_MAX_ROWS];

constexpr int kMaxDevices = 64;
float* g_delta_ptr[kMaxDevices] = {nullptr};

int fail(char* err, int err_len, int code, const char* msg) {
  if (err != nullptr && err_len > 0) {
    std::strncpy(err, msg, (size_t)err_len - 1);
    err[err_len - 1] = '\0';
  }
  return code;
}

}  // namespace

extern "C" int zx_attn_bwd_noalloc(const void* q, const void* k, const void* v, const void* o, const void* d_o,
                                   const float* lse, float* dq, float* dk, float* dv, int B, int Hq, int Hkv, int Sq,
                                   int Skv, long long q_tok_stride, long long k_tok_stride, long long v_tok_stride,
                                   float scale, int causal, int* status_out, void* stream, char* err, int err_len) {
  char msg[256];
  if (q == nullptr || k == nullptr || v == nullptr || o == nullptr || d_o == nullptr || lse == nullptr ||
      dq == nullptr || dk == nullptr || dv == nullptr)
    return fail(err, err_len, 1, "zx_attn_bwd_noalloc: null pointer argument");
  if (B <= 0 || Hq <= 0 || Hkv <= 0 || Sq <= 0 || Skv <= 0)
    return fail(err, err_len, 1, "zx_attn_bwd_noalloc: sizes must be positive");
  const long long rows = (long long)B * Hq * Sq;
  if (rows > (long long)ZX_ATTN_BWD_NOALLOC_MAX_ROWS) {
    std::snprintf(msg, sizeof(msg),
                  "zx_attn_bwd_noalloc: B*Hq*Sq = %lld exceeds the built-in scratch of %d rows; "
                  "use the regular backward with a caller-allocated delta buffer",
                  rows, (int)ZX_ATTN_BWD_NOALLOC_MAX_ROWS);
    return fail(err, err_len, 2, msg);
  }
  // Everything that can reject the call is checked before anything of the caller's is written.
  if (Sq % 128 != 0 || Skv % 128 != 0)
    return fail(err, err_len, 1, "zx_attn_bwd_noalloc: Sq and Skv must be multiples of 128");
  if (Hq % Hkv != 0) return fail(err, err_len, 1, "zx_attn_bwd_noalloc: Hq must be a multiple of Hkv");
  if (q_tok_stride < (long long)Hq * 128 || k_tok_stride < (long long)Hkv * 128 || v_tok_stride < (long long)Hkv * 128 ||
      q_tok_stride % 8 != 0 || k_tok_stride % 8 != 0 || v_tok_stride % 8 != 0)
    return fail(err, err_len, 1,
                "zx_attn_bwd_noalloc: token strides must cover all heads and be multiples of 8 elements (16 bytes)");
  if (((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)o | (uintptr_t)d_o | (uintptr_t)dq | (uintptr_t)dk |
       (uintptr_t)dv) % 16 != 0)
    return fail(err, err_len, 1, "zx_attn_bwd_noalloc: tensor pointers must be 16-byte aligned");
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices)
    return fail(err, err_len, 3, "zx_attn_bwd_noalloc: cannot determine the current device");
  if (g_delta_ptr[dev] == nullptr) {
    // once per device, with that device current
    float* p = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_delta_scratch);
    if (e != cudaSuccess || p == nullptr) {
      std::snprintf(msg, sizeof(msg), "zx_attn_bwd_noalloc: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
      return fail(err, err_len, 3, msg);
    }
    g_delta_ptr[dev] = p;
  }
  // An error left behind by an earlier, unrelated call must not be blamed on this launch.
  const cudaError_t pending = cudaPeekAtLastError();
  if (pending != cudaSuccess) {
    std::snprintf(msg, sizeof(msg), "zx_attn_bwd_noalloc: an earlier CUDA error is pending on this thread: %s",
                  cudaGetErrorString(pending));
    return fail(err, err_len, 7, msg);
  }
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const size_t kv_bytes = (size_t)B * Skv * Hkv * 128 * sizeof(float);
  if ((e = cudaMemsetAsync(dk, 0, kv_bytes, st)) != cudaSuccess || (e = cudaMemsetAsync(dv, 0, kv_bytes, st)) != cudaSuccess ||
      (status_out != nullptr && (e = cudaMemsetAsync(status_out, 0, sizeof(zx::Status), st)) != cudaSuccess)) {
    std::snprintf(msg, sizeof(msg), "zx_attn_bwd_noalloc: clearing the outputs failed: %s", cudaGetErrorString(e));
    return fail(err, err_len, 4, msg);
  }
  try {
    zx::AttnBwdArgs a;
    a.q = q; a.k = k; a.v = v; a.o = o; a.d_o = d_o;
    a.lse = lse;
    a.delta = g_delta_ptr[dev];
    a.dq = dq; a.dk = dk; a.dv = dv;
    a.B = B; a.Hq = Hq; a.Hkv = Hkv; a.Sq = Sq; a.Skv = Skv;
    a.q_tok_stride = q_tok_stride; a.k_tok_stride = k_tok_stride; a.v_tok_stride = v_tok_stride;
    a.scale = scale;
    a.mask.causal = causal ? 1 : 0;
    a.q_layout.n_chunks = 1; a.q_layout.chunk_len = Sq; a.q_layout.chunk_pos[0] = 0;
    a.kv_layout.n_chunks = 1; a.kv_layout.chunk_len = Skv; a.kv_layout.chunk_pos[0] = 0;
    a.compute_delta = 1;
    a.dq_accumulate = 0;
    a.status = reinterpret_cast<zx::Status*>(status_out);
    a.stream = st;
    zx::launch_attn_bwd(a);
  } catch (const std::exception& ex) {
    return fail(err, err_len, 5, ex.what());
  }
  e = cudaGetLastError();
  if (e != cudaSuccess) {
    std::snprintf(msg, sizeof(msg), "zx_attn_bwd_noalloc: launch failed: %s", cudaGetErrorString(e));
    return fail(err, err_len, 6, msg);
  }
  return 0;
}
