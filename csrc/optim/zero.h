// Sharded AdamW fused with its collectives over peer memory (launch interface).
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>
#include "../common/status.h"
#include "../peer/peer.h"

namespace zx {

struct ZeroArgs {
  // Flat parameter space of n_total elements; this rank owns [shard_begin, shard_begin + n_shard).
  // All counts are multiples of 4.
  PeerPtrs grads;    // every rank's fp32 gradient buffer [n_total] (peer-mapped; index = rank)
  PeerPtrs params;   // every rank's bf16 parameter buffer [n_total] (peer-mapped)
  int nranks = 1;
  int rank = 0;
  size_t shard_begin = 0;
  size_t n_shard = 0;
  size_t decay_end = 0;   // weight decay applies to global indices < decay_end
  // local shard state
  float* g_shard = nullptr;    // [n_shard] reduced gradient (written in reduce mode, read in update mode)
  int16_t* p_lo = nullptr;     // [n_shard]
  void* m = nullptr;           // [n_shard] fp32, or bf16 when state_bf16
  void* v = nullptr;           // [n_shard]
  int state_bf16 = 0;          // Adam's moments are stored as bf16 (arithmetic stays fp32; the master weight is unaffected)
  float* sumsq = nullptr;      // [1] accumulates the squared norm of the reduced shard (reduce mode)
  const float* clip_coef = nullptr;  // [1] optional device-side factor applied to the gradient
  int do_reduce = 1;           // sum the shard over all ranks' gradient buffers (P2P loads)
  int do_update = 1;           // AdamW + push of the new bf16 parameters to every rank (P2P stores)
  int zero_grads = 0;          // clear this rank's slice of every rank's gradient buffer after reading
  float grad_scale = 1.f;      // e.g. 1 / (accumulation steps * data-parallel replicas)
  float lr = 0.f, beta1 = 0.9f, beta2 = 0.95f, eps = 1e-8f, weight_decay = 0.f;
  int step = 1;
  int sm_count = 148;
  cudaStream_t stream = nullptr;
};

void launch_zero_step(const ZeroArgs& args);

}  // namespace zx
