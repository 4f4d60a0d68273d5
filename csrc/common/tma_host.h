// Host-side construction of TMA tensor maps without linking libcuda: the driver entry point is
// looked up through the runtime, so the library still loads on a machine with no driver.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdexcept>
#include <string>

namespace zx {

typedef CUresult (*PFN_encodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline PFN_encodeTiled get_encode_tiled() {
  static PFN_encodeTiled fn = nullptr;
  if (fn) return fn;
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q);
  if (e != cudaSuccess || p == nullptr || q != cudaDriverEntryPointSuccess)
    throw std::runtime_error("zenyx_b200: cuTensorMapEncodeTiled is not available (no CUDA driver?)");
  fn = reinterpret_cast<PFN_encodeTiled>(p);
  return fn;
}

enum class TmaSwizzle { None, B128 };

// Generic tiled map, up to rank 4. dims[0] is the contiguous dimension. strides_bytes[i] is the
// byte stride of dims[i+1] (rank-1 entries), each a multiple of 16. box[0]*elem_size must be
// <= 128 bytes when 128B swizzle is used.
inline CUtensorMap make_tma_map(const void* base, int elem_bytes, int rank, const uint64_t* dims,
                                const uint64_t* strides_bytes, const uint32_t* box, TmaSwizzle swz) {
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0) throw std::runtime_error("TMA base must be 16-byte aligned");
  for (int i = 0; i + 1 < rank; ++i)
    if (strides_bytes[i] % 16 != 0) throw std::runtime_error("TMA strides must be multiples of 16 bytes");
  CUtensorMap m;
  cuuint64_t gdims[5];
  cuuint64_t gstr[5];
  cuuint32_t bx[5];
  cuuint32_t es[5];
  for (int i = 0; i < rank; ++i) {
    gdims[i] = dims[i];
    bx[i] = box[i];
    es[i] = 1;
    if (i + 1 < rank) gstr[i] = strides_bytes[i];
  }
  CUtensorMapDataType dt = elem_bytes == 2   ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                           : elem_bytes == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                             : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  CUresult r = get_encode_tiled()(&m, dt, (cuuint32_t)rank, const_cast<void*>(base), gdims, gstr, bx, es,
                                  CU_TENSOR_MAP_INTERLEAVE_NONE,
                                  swz == TmaSwizzle::B128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) throw std::runtime_error("cuTensorMapEncodeTiled failed with code " + std::to_string((int)r));
  return m;
}

// 2-D row-major matrix [rows, cols] with leading dimension ld (elements).
inline CUtensorMap make_tma_2d(const void* base, int elem_bytes, uint64_t rows, uint64_t cols, uint64_t ld,
                               uint32_t box_cols, uint32_t box_rows) {
  uint64_t dims[2] = {cols, rows};
  uint64_t str[1] = {ld * (uint64_t)elem_bytes};
  uint32_t box[2] = {box_cols, box_rows};
  return make_tma_map(base, elem_bytes, 2, dims, str, box, TmaSwizzle::B128);
}

}  // namespace zx
