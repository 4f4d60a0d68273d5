// CUDA IPC plumbing for peer-visible buffers: one process per GPU allocates with cudaMalloc,
// exports the handle, and every other rank of the node maps it. The mapped pointers are then used
// directly by kernels (P2P loads / stores / reductions over NVLink); no library kernel is ever
// given such a pointer.
#include <cuda_runtime.h>
#include <cstring>
#include <stdexcept>
#include <string>
#include "peer.h"

namespace zx {

static void check(cudaError_t e, const char* what) {
  if (e != cudaSuccess) throw std::runtime_error(std::string("peer memory: ") + what + ": " + cudaGetErrorString(e));
}

void* peer_alloc(size_t bytes) {
  void* p = nullptr;
  check(cudaMalloc(&p, bytes), "cudaMalloc");
  check(cudaMemset(p, 0, bytes), "cudaMemset");
  check(cudaDeviceSynchronize(), "sync after clear");
  return p;
}

std::string peer_export(void* ptr) {
  cudaIpcMemHandle_t h;
  check(cudaIpcGetMemHandle(&h, ptr), "cudaIpcGetMemHandle");
  return std::string(reinterpret_cast<const char*>(&h), sizeof(h));
}

void* peer_open(const std::string& handle) {
  if (handle.size() != sizeof(cudaIpcMemHandle_t)) throw std::runtime_error("peer memory: bad handle size");
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle.data(), sizeof(h));
  void* p = nullptr;
  check(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle");
  return p;
}

void peer_close(void* mapped) { check(cudaIpcCloseMemHandle(mapped), "cudaIpcCloseMemHandle"); }

void peer_free(void* ptr) { check(cudaFree(ptr), "cudaFree"); }

}  // namespace zx
