// Launch interface of the tcgen05 bf16 GEMM (no torch types: raw pointers and a stream).
#pragma once
#include <cuda_runtime.h>
#include "../common/status.h"

namespace zx {

struct GemmArgs {
  // C[M,N] = A * B^T (+ D).  Logical A is M x K, logical B is N x K.
  // a_mn == false: A stored row-major [M, K] with leading dimension lda.
  // a_mn == true : A stored row-major [K, M] (i.e. transposed), leading dimension lda.
  // Same for B / b_mn with N in place of M.
  const void* A = nullptr;
  const void* B = nullptr;
  void* C = nullptr;
  const void* D = nullptr;  // optional addend with the shape of C (may alias C)
  int M = 0, N = 0, K = 0;
  int lda = 0, ldb = 0, ldc = 0, ldd = 0;
  bool a_mn = false, b_mn = false;
  int out_fp32 = 0;  // C is fp32 instead of bf16
  int d_mode = 0;    // 0: no addend, 1: bf16 addend, 2: fp32 addend
  Status* status = nullptr;
  cudaStream_t stream = nullptr;
  int sm_count = 148;
};

void launch_gemm_bf16(const GemmArgs& args);

}  // namespace zx
