// Kernels that talk to peer GPUs directly: the flag barrier and an SM-issued pull copy.
#include "../common/ptx.cuh"
#include "peer.h"

namespace zx {

namespace {

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__global__ void peer_barrier_kernel(PeerPtrs flags, int rank, int nranks, uint32_t epoch, uint64_t timeout_ns,
                                    Status* status) {
  const int t = threadIdx.x;
  if (t < nranks) {
    __threadfence_system();  // everything this GPU wrote before the barrier is visible to peers first
    st_release_sys(reinterpret_cast<uint32_t*>(flags.p[t]) + rank, epoch);
    const uint32_t* mine = reinterpret_cast<const uint32_t*>(flags.p[rank]) + t;
    const uint64_t t0 = globaltimer_ns();
    bool ok = false;
    while (true) {
      // epochs only grow; the signed difference tolerates wrap-around
      if ((int32_t)(ld_acquire_sys(mine) - epoch) >= 0) { ok = true; break; }
      if (globaltimer_ns() - t0 > timeout_ns) break;
      __nanosleep(200);
    }
    if (!ok) report(status, ZX_ERR_TIMEOUT, /*site=*/31, t);
  }
}

__global__ void peer_pull_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, size_t nvec) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (size_t)gridDim.x * blockDim.x) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(src + i));
    dst[i] = v;
  }
}

}  // namespace

void launch_peer_barrier(const PeerPtrs& flags, int rank, int nranks, uint32_t epoch, uint64_t timeout_ns,
                         Status* status, cudaStream_t stream) {
  peer_barrier_kernel<<<1, 32, 0, stream>>>(flags, rank, nranks, epoch, timeout_ns, status);
}

void launch_peer_pull(const void* src_peer, void* dst_local, size_t bytes, int blocks, cudaStream_t stream) {
  if (bytes == 0) return;
  peer_pull_kernel<<<blocks, 256, 0, stream>>>((const uint4*)src_peer, (uint4*)dst_local, bytes / 16);
}

}  // namespace zx
