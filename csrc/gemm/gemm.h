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
  // Fused all-gather: while the tiles compute, one extra warp per CTA copies this CTA's slice of a
  // (possibly peer-resident) buffer into local memory with plain 16-byte loads, so the operand of
  // the NEXT launch crosses NVLink underneath this launch's math. Sizes in bytes, multiples of 16.
  const void* pull_src = nullptr;
  void* pull_dst = nullptr;
  size_t pull_bytes = 0;
  // Fused reduce-scatter, first half: instead of one C, every row block is STORED (bf16) into the
  // receive slot that its owner keeps for this rank: row m goes to
  //   scatter_base[m / rows_per_rank] + (scatter_src_rank * rows_per_rank + m % rows_per_rank) * ldc.
  // The bases are peer-mapped pointers, so the partial tiles cross NVLink as the accumulators drain;
  // after a barrier the owner sums its `scatter_ranks` slots (sum_slots_bf16).
  int scatter_ranks = 0;
  int scatter_rows_per_rank = 0;
  int scatter_src_rank = 0;
  void* scatter_base[8] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
  Status* status = nullptr;
  cudaStream_t stream = nullptr;
  int sm_count = 148;
};

void launch_gemm_bf16(const GemmArgs& args);

}  // namespace zx
