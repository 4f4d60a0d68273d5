// Thin inline-PTX layer for sm_100a: mbarrier, TMA (per-CTA loads only), tcgen05 MMA / TMEM.
// Everything here is header-only and free of torch includes so kernels compile in seconds.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <type_traits>
#include "status.h"

namespace zx {

__device__ __forceinline__ void report(Status* st, int code, int site, int info) {
  if (st == nullptr) return;
  if (atomicCAS(&st->code, ZX_OK, code) == ZX_OK) {
    st->site = site;
    st->block = (int)blockIdx.x;
    st->info = info;
  }
}

// Checked build (-DZX_CHECKED, `python -m zenyx_b200._build --checked`): the index of every global-memory row a
// kernel epilogue writes is compared with its extent first; a bad index is recorded in the status word
// (ZX_ERR_BOUNDS with the site and the index) and the access is skipped, so the context stays usable and the
// host reads what went wrong. In normal builds the macro is the constant `true` and costs nothing.
#ifdef ZX_CHECKED
#define ZX_IN_BOUNDS(st, idx, limit, site) \
  ((unsigned long long)(idx) < (unsigned long long)(limit) ? true : (::zx::report((st), ::zx::ZX_ERR_BOUNDS, (site), (int)(idx)), false))
#else
#define ZX_IN_BOUNDS(st, idx, limit, site) true
#endif

// ----------------------------------------------------------------------------------------------
// Basic helpers
// ----------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred = 0;
  asm volatile(
      "{\n\t"
      ".reg .pred P;\n\t"
      "elect.sync _|P, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, P;\n\t"
      "}\n"
      : "=r"(pred));
  return pred != 0;
}

// ----------------------------------------------------------------------------------------------
// mbarrier
// ----------------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// One arrival per warp: an arrive is an atomic on one shared-memory word, so 32 lanes arriving
// separately serialise (a 512-thread arrival costs over a thousand cycles of the item's critical
// path). The warp converges first, which also orders every lane's earlier writes before the
// single arrive. Barriers used with this are initialised with their WARP count.
__device__ __forceinline__ void mbar_arrive_warp(uint64_t* bar) {
  __syncwarp();
  if ((threadIdx.x & 31) == 0) mbar_arrive(bar);
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred P;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, P;\n\t"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Wait limit for in-kernel waits. All producers of these barriers live in the same kernel, so a
// healthy wait is microseconds; two seconds only ever elapses when the protocol is broken.
#ifndef ZX_WAIT_LIMIT_NS
#define ZX_WAIT_LIMIT_NS 2000000000ull
#endif

// Bounded wait. Returns false when the wait gave up (its own limit, or another role already
// raised *abort). The caller must then fall through to the kernel's teardown.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
#pragma unroll 1
  for (int i = 0; i < 1024; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
  }
  const uint64_t t0 = globaltimer_ns();
#pragma unroll 1
  while (true) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i) {
      if (mbar_try_wait(bar, parity)) return true;
    }
    if (*abort_flag) return false;
    if (globaltimer_ns() - t0 > ZX_WAIT_LIMIT_NS) {
      *abort_flag = 1;
      return false;
    }
  }
}

__device__ __forceinline__ bool mbar_wait_w(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  const bool ok = mbar_wait(bar, parity, abort_flag);
  return __all_sync(0xffffffffu, ok);
}

// ----------------------------------------------------------------------------------------------
// TMA (tiled bulk tensor copies). Every load targets the issuing CTA only.
// ----------------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* m, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* m, uint64_t* bar, int x, int y,
                                            int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z)
      : "memory");
}
__device__ __forceinline__ void tma_load_4d(void* smem_dst, const CUtensorMap* m, uint64_t* bar, int x, int y,
                                            int z, int w) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], "
      "[%2];" ::"r"(smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z), "r"(w)
      : "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* m, const void* smem_src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(m)),
               "r"(smem_u32(smem_src)), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void tma_store_wait() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// ----------------------------------------------------------------------------------------------
// tcgen05: TMEM allocation, MMA, commit, TMEM <-> register moves
// ----------------------------------------------------------------------------------------------
// One full warp allocates `ncols` (power of two, 32..512) columns; the base address lands in smem.
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// D[tmem] (+)= A[smem desc] * B[smem desc]; bf16/fp16 inputs, fp32 accumulate. One thread issues.
__device__ __forceinline__ void umma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Same with the A operand read from TMEM (M x K, two 16-bit values per 32-bit column).
__device__ __forceinline__ void umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
      "}\n" ::"r"(d_tmem),
      "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// fp8 (e4m3/e5m2) inputs, fp32 accumulate; K per instruction is 32.
__device__ __forceinline__ void umma_ss_f8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t"
      "}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Warp-collective forms: every lane of a converged warp executes the statement, one elected lane
// (always the same one for a full warp) issues the instruction. Keeping the MMA warp's control
// flow uniform lets the compiler hold descriptors and addresses in uniform registers, which is
// what tcgen05.mma consumes; issuing from inside an `if (lane == 0)` branch costs a register
// transfer per operand per instruction.
__device__ __forceinline__ void umma_ss_w(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p, e;\n\t"
      "elect.sync _|e, 0xffffffff;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_ts_w(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p, e;\n\t"
      "elect.sync _|e, 0xffffffff;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
      "}\n" ::"r"(d_tmem),
      "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit_w(uint64_t* bar) {
  asm volatile(
      "{\n\t"
      ".reg .pred e;\n\t"
      "elect.sync _|e, 0xffffffff;\n\t"
      "@e tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t"
      "}\n" ::"r"(smem_u32(bar))
      : "memory");
}
// Eight MMAs of one 128 x N x 128 product (K = 8 x 16) in ONE asm statement: one election, the per-step
// descriptor offsets as immediates. The issuing warp's instruction stream is on the critical path of the
// attention kernels (it competes for issue slots with the softmax warps of its scheduler), so the cost per
// MMA has to stay at a few instructions.
//  K-major operand stored as two 64-element halves (HALF16 = distance of the halves in 16-byte units):
//    step k starts at (k / 4) * HALF16 + (k % 4) * 2
//  MN-major operand (rows = K index, 128 bytes per row): step k starts at k * 16 rows = k * 128 units.
template <int HALF16>
__device__ __forceinline__ void umma_ss_k8_kmajor_w(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                    uint32_t acc_first) {
  asm volatile(
      "{\n\t"
      ".reg .pred e, p, t;\n\t"
      ".reg .b64 a, b;\n\t"
      "elect.sync _|e, 0xffffffff;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "setp.eq.b32 t, %3, %3;\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "add.s64 a, %1, 2;\n\t add.s64 b, %2, 2;\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %3, t;\n\t"
      "add.s64 a, %1, 4;\n\t add.s64 b, %2, 4;\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %3, t;\n\t"
      "add.s64 a, %1, 6;\n\t add.s64 b, %2, 6;\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %3, t;\n\t"
      "add.s64 a, %1, %5;\n\t add.s64 b, %2, %5;\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %3, t;\n\t"
      "add.s64 a, %1, %6;\n\t add.s64 b, %2, %6;\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %3, t;\n\t"
      "add.s64 a, %1, %7;\n\t add.s64 b, %2, %7;\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %3, t;\n\t"
      "add.s64 a, %1, %8;\n\t add.s64 b, %2, %8;\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %3, t;\n\t"
      "}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(acc_first), "n"(HALF16), "n"(HALF16 + 2), "n"(HALF16 + 4),
      "n"(HALF16 + 6)
      : "memory");
}
// A (M x 128 bf16, two values per 32-bit column) read from TMEM, B MN-major in shared memory. A1..A7 are the
// TMEM column offsets of K steps 1..7 relative to step 0 (8 columns per step when A is stored contiguously;
// the backward kernels keep it in several column groups).
template <int A1, int A2, int A3, int A4, int A5, int A6, int A7>
__device__ __forceinline__ void umma_ts_k8_w(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                             uint32_t acc_first) {
  asm volatile(
      "{\n\t"
      ".reg .pred e, p, t;\n\t"
      ".reg .b32 ta;\n\t"
      ".reg .b64 b;\n\t"
      "elect.sync _|e, 0xffffffff;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "setp.eq.b32 t, %3, %3;\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
      "add.u32 ta, %1, %5;\n\t add.s64 b, %2, 128;\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [ta], b, %3, t;\n\t"
      "add.u32 ta, %1, %6;\n\t add.s64 b, %2, 256;\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [ta], b, %3, t;\n\t"
      "add.u32 ta, %1, %7;\n\t add.s64 b, %2, 384;\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [ta], b, %3, t;\n\t"
      "add.u32 ta, %1, %8;\n\t add.s64 b, %2, 512;\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [ta], b, %3, t;\n\t"
      "add.u32 ta, %1, %9;\n\t add.s64 b, %2, 640;\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [ta], b, %3, t;\n\t"
      "add.u32 ta, %1, %10;\n\t add.s64 b, %2, 768;\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [ta], b, %3, t;\n\t"
      "add.u32 ta, %1, %11;\n\t add.s64 b, %2, 896;\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [ta], b, %3, t;\n\t"
      "}\n" ::"r"(d_tmem),
      "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(acc_first), "n"(A1), "n"(A2), "n"(A3), "n"(A4), "n"(A5), "n"(A6), "n"(A7)
      : "memory");
}
__device__ __forceinline__ void umma_ts_k8_mnmajor_w(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                                     uint32_t acc_first) {
  umma_ts_k8_w<8, 16, 24, 32, 40, 48, 56>(d_tmem, a_tmem, b_desc, idesc, acc_first);
}
// Half of the above: four MMAs (K = 4 x 16 = 64), so that P V can start on the first 64 probabilities of a
// row block while the softmax warps still work on the other 64.
__device__ __forceinline__ void umma_ts_k4_mnmajor_w(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                                     uint32_t acc_first) {
  asm volatile(
      "{\n\t"
      ".reg .pred e, p, t;\n\t"
      ".reg .b32 ta;\n\t"
      ".reg .b64 b;\n\t"
      "elect.sync _|e, 0xffffffff;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "setp.eq.b32 t, %3, %3;\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
      "add.u32 ta, %1, 8;\n\t add.s64 b, %2, 128;\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [ta], b, %3, t;\n\t"
      "add.u32 ta, %1, 16;\n\t add.s64 b, %2, 256;\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [ta], b, %3, t;\n\t"
      "add.u32 ta, %1, 24;\n\t add.s64 b, %2, 384;\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [ta], b, %3, t;\n\t"
      "}\n" ::"r"(d_tmem),
      "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(acc_first)
      : "memory");
}
// Warp-uniform bounded wait: every lane polls, the verdict is shared.
__device__ __forceinline__ bool mbar_wait_w(uint64_t* bar, uint32_t parity, volatile int* abort_flag);

// Arrive on an mbarrier once every MMA issued so far by this thread has finished.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

// TMEM address = (lane << 16) | column.
__device__ __forceinline__ uint32_t tmem_addr(uint32_t base, uint32_t lane, uint32_t col) {
  return base + (lane << 16) + col;
}

// 32 lanes x 32 bit, 32 consecutive columns: thread t of the warp gets lane (warp%4)*32+t.
__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_32x32b_x16(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st_32x32b_x32(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
      "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]),
      "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]),
      "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_32x32b_x16(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
      "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}

// 16 lanes x 256 bit per repeat: the accumulator-fragment layout. With lane base L (a multiple of 16 inside the
// warp's lane quarter) thread t holds, for repeat k, r[4k], r[4k+1] = lane L + t/4, columns 8k + 2(t%4), +1 and
// r[4k+2], r[4k+3] = lane L + t/4 + 8, same columns. A row is spread over four neighbouring threads, so two
// warps can share a lane quarter by rows (16 each) and reduce along a row with two shuffles.
__device__ __forceinline__ void tmem_ld_16x256b_x16(uint32_t taddr, uint32_t* r) {
  asm volatile("tcgen05.ld.sync.aligned.16x256b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, %48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%64];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31]), "=r"(r[32]), "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]), "=r"(r[37]), "=r"(r[38]), "=r"(r[39]), "=r"(r[40]), "=r"(r[41]), "=r"(r[42]), "=r"(r[43]), "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47]), "=r"(r[48]), "=r"(r[49]), "=r"(r[50]), "=r"(r[51]), "=r"(r[52]), "=r"(r[53]), "=r"(r[54]), "=r"(r[55]), "=r"(r[56]), "=r"(r[57]), "=r"(r[58]), "=r"(r[59]), "=r"(r[60]), "=r"(r[61]), "=r"(r[62]), "=r"(r[63])
               : "r"(taddr)
               : "memory");
}
__device__ __forceinline__ void tmem_ld_16x256b_x8(uint32_t taddr, uint32_t* r) {
  asm volatile("tcgen05.ld.sync.aligned.16x256b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
               : "r"(taddr)
               : "memory");
}
__device__ __forceinline__ void tmem_st_16x256b_x8(uint32_t taddr, const uint32_t* r) {
  asm volatile("tcgen05.st.sync.aligned.16x256b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
               : "memory");
}
// 16 lanes x 128 bit per repeat: thread t holds r[2k] = lane L + t/4, column 4k + t%4 and r[2k+1] = lane L + t/4 + 8,
// same column: the packed-pair counterpart of the layout above.
__device__ __forceinline__ void tmem_st_16x128b_x8(uint32_t taddr, const uint32_t* r) {
  asm volatile("tcgen05.st.sync.aligned.16x128b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
               : "memory");
}

// Register re-balancing between warpgroups (all four warps of a warpgroup must execute it).
template <int N>
__device__ __forceinline__ void setmaxnreg_inc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N>
__device__ __forceinline__ void setmaxnreg_dec() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}

// ----------------------------------------------------------------------------------------------
// Descriptors
// ----------------------------------------------------------------------------------------------
// Shared-memory matrix descriptor, 128-byte swizzle. Tiles are stored as rows of 128 bytes
// (64 bf16 / 128 fp8), eight rows per 1024-byte swizzle atom, base 1024-byte aligned.
//  K-major  operand: row = M/N index, the 128 bytes run along K.  sbo = 1024 (next 8 rows).
//  MN-major operand: row = K index, the 128 bytes run along M/N.  sbo = 1024 (next 8 K rows),
//                    lbo = byte distance between consecutive 64-element (128 B) chunks along M/N.
__device__ __forceinline__ uint64_t make_smem_desc_sw128(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;  // descriptor version (Blackwell)
  d |= (uint64_t)2 << 61;  // SWIZZLE_128B
  return d;
}

// Byte offset applied to a descriptor's start-address field (the field holds address >> 4 and the
// tiles used here never carry out of it), so per-k-step descriptors cost one add.
__device__ __forceinline__ uint64_t desc_advance(uint64_t d, uint32_t bytes) { return d + (uint64_t)(bytes >> 4); }

// Instruction descriptor for kind::f16 (fmt: 0 = fp16, 1 = bf16) / kind::f8f6f4 (fmt: 0 = e4m3, 1 = e5m2)
// with fp32 accumulation. a_mn / b_mn: 1 when that operand is MN-major in shared memory.
__host__ __device__ constexpr uint32_t make_idesc(int M, int N, int a_fmt, int b_fmt, int a_mn, int b_mn) {
  return (1u << 4) | ((uint32_t)a_fmt << 7) | ((uint32_t)b_fmt << 10) | ((uint32_t)a_mn << 15) |
         ((uint32_t)b_mn << 16) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

// ----------------------------------------------------------------------------------------------
// Fused peer pull: one warp copies this CTA's slice of a (possibly remote) buffer into local
// memory with 16-byte loads, several in flight per lane. Sizes are in 16-byte vectors.
// ----------------------------------------------------------------------------------------------
__device__ __forceinline__ uint4 ld_stream_v4(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
// DEPTH 16-byte loads are in flight per lane: a peer load takes about 2 us over NVLink, so the copy rate of
// one warp is DEPTH * 32 * 16 B per round trip, and 148 such warps need DEPTH >= 8 to keep up with a GEMM or
// attention launch of a few hundred microseconds.
template <int DEPTH = 8>
__device__ __forceinline__ void warp_pull_slice(const uint4* __restrict__ src, uint4* __restrict__ dst, size_t nvec,
                                                int lane) {
  if (src == nullptr || nvec == 0) return;
  const size_t per = (nvec + gridDim.x - 1) / gridDim.x;
  const size_t begin = (size_t)blockIdx.x * per;
  size_t end = begin + per;
  if (end > nvec) end = nvec;
  size_t i = begin + lane;
  for (; i + 32 * (DEPTH - 1) < end; i += 32 * DEPTH) {
    uint4 v[DEPTH];
#pragma unroll
    for (int k = 0; k < DEPTH; ++k) v[k] = ld_stream_v4(src + i + 32 * k);
#pragma unroll
    for (int k = 0; k < DEPTH; ++k) dst[i + 32 * k] = v[k];
  }
  for (; i < end; i += 32) dst[i] = ld_stream_v4(src + i);
}

// Compile-time loop: f(std::integral_constant<int, i>) for i in [0, N).
template <int N, int I = 0, typename F>
__device__ __forceinline__ void static_for(F&& f) {
  if constexpr (I < N) {
    f(std::integral_constant<int, I>{});
    static_for<N, I + 1>(f);
  }
}

// ----------------------------------------------------------------------------------------------
// Small numeric helpers
// ----------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float2 unpack_bf16x2(uint32_t u) {
  __nv_bfloat162 v = *reinterpret_cast<__nv_bfloat162*>(&u);
  return __bfloat1622float2(v);
}
// max of three in one instruction
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// 2^x for two values on the FMA pipe instead of the special-function unit. The unit produces 16
// results per clock per SM, which is what bounds a softmax tile once the rest of the row's
// arithmetic is packed; moving a quarter of the exponentials here balances the two pipes.
// x = j + f with j = round(x), |f| <= 1/2; 2^f by a cubic fitted on [-1/2, 1/2] (relative error
// below 8e-5, far inside the bf16 rounding the result gets) and j goes straight into the exponent
// field. Inputs below -125 return (almost) zero.
__device__ __forceinline__ float2 exp2_poly2(float2 x) {
  x.x = fmaxf(x.x, -125.f);
  x.y = fmaxf(x.y, -125.f);
  const float2 t = __fadd2_rn(x, make_float2(12582912.f, 12582912.f));   // 1.5 * 2^23: round(x) lands in the mantissa
  const float2 j = __fadd2_rn(t, make_float2(-12582912.f, -12582912.f));
  const float2 f = __fadd2_rn(x, make_float2(-j.x, -j.y));
  float2 q = __ffma2_rn(f, make_float2(0.05517166f, 0.05517166f), make_float2(0.24261113f, 0.24261113f));
  q = __ffma2_rn(q, f, make_float2(0.69326097f, 0.69326097f));
  q = __ffma2_rn(q, f, make_float2(0.99992806f, 0.99992806f));
  return make_float2(__int_as_float((__float_as_int(t.x) << 23) + __float_as_int(q.x)),
                     __int_as_float((__float_as_int(t.y) << 23) + __float_as_int(q.y)));
}
// Pair exponential; every kEvery-th pair (by the caller's compile-time index) takes the FMA pipe. Four suits a
// loop whose FMA pipe is already busy (the forward softmax: row sums, packing); two suits the backward kernels,
// whose exponential phase sits alone on the critical path with the FMA pipe nearly idle.
template <int kIndex, int kEvery = 4>
__device__ __forceinline__ float2 exp2_pair(float2 x) {
#ifndef ZX_NO_POLY
  if ((kIndex % kEvery) == kEvery - 1) return exp2_poly2(x);
#endif
  return make_float2(fast_exp2(x.x), fast_exp2(x.y));
}

}  // namespace zx
