// Peer (symmetric) memory over CUDA IPC and the kernels that work on it directly.
// The reference has no counterpart: its only transport is torch.distributed
// (zenyx/distributed/communication.py:136-171).
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>
#include <string>
#include "../common/status.h"

namespace zx {

constexpr int kMaxPeers = 8;

// --- host side (ipc_memory.cpp) ---
void* peer_alloc(size_t bytes);                       // cudaMalloc'ed and zeroed, exportable
std::string peer_export(void* ptr);                   // opaque IPC handle bytes
void* peer_open(const std::string& handle);           // maps a peer's allocation into this process
void peer_close(void* mapped);
void peer_free(void* ptr);

struct PeerPtrs {
  void* p[kMaxPeers];
};

// --- kernels (peer_kernels.cu) ---
// Flag barrier over peer memory: every rank stores `epoch` into slot `rank` of each peer's flag
// array, then waits (bounded by timeout_ns) until its own array shows `epoch` from all ranks.
void launch_peer_barrier(const PeerPtrs& flags, int rank, int nranks, uint32_t epoch, uint64_t timeout_ns,
                         Status* status, cudaStream_t stream);

// Plain peer copy issued from SMs (ld from the peer over NVLink, st locally).
void launch_peer_pull(const void* src_peer, void* dst_local, size_t bytes, int blocks, cudaStream_t stream);

}  // namespace zx
