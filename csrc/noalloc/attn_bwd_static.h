// Attention backward for callers that cannot allocate device memory.
//
// This entry point has no counterpart in the reference project (which ships no native code).
//
// Who needs it: code that runs where cudaMalloc is off limits - a plugin or callback that is only
// handed raw device pointers and a stream and does not own an allocator, a host that pre-commits
// all of its device memory at start-up and forbids later growth, or a latency-critical loop where
// an allocation (and the implicit device synchronisation it can bring) is not acceptable. The
// regular backward (`launch_attn_bwd`) needs one scratch buffer, delta = rowsum(dO * O) with
// B * Hq * Sq floats, which its callers allocate. Here that scratch lives in a fixed array inside
// the library instead, so the caller passes only inputs and outputs.
//
// Limits and rules:
//  * B * Hq * Sq must not exceed ZX_ATTN_BWD_NOALLOC_MAX_ROWS (1,048,576 rows = 4 MiB of scratch,
//    e.g. one 32768-token sequence with 32 query heads). Larger problems are rejected with an error
//    message; nothing is launched. Every GPU that loads the library holds those 4 MiB until exit.
//  * The first call on a device resolves the scratch array's device address and raises the
//    kernels' shared-memory limit. Make that first call outside of any stream capture.
//  * All calls share the one scratch array (it keeps the previous call's contents; the kernels
//    overwrite every element they later read, so nothing needs clearing there). Two calls that
//    may overlap on the GPU - different streams without an ordering between them - race on it.
//    Calls on one stream are safe.
//  * dk and dv are cleared by this function (the kernels accumulate into them); dq is overwritten.
//  * No cudaMalloc / cudaFree and no allocating library routine is called.
//
// Layout: q [B,Sq,Hq,128] and k, v [B,Skv,Hkv,128] are bf16 with the given token strides (in
// elements); o and d_o are contiguous bf16 [B,Sq,Hq,128]; lse is fp32 [B,Hq,Sq] from the forward;
// dq [B,Sq,Hq,128], dk and dv [B,Skv,Hkv,128] are contiguous fp32. Token positions are 0..S-1.
// status_out, if not null, points to 4 ints of device memory that receive the kernels' status
// word (all zero = success; it is cleared first). Returns 0 on success; otherwise a non-zero code
// and, if err is not null, a message of at most err_len - 1 characters.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

#define ZX_ATTN_BWD_NOALLOC_MAX_ROWS (1 << 20)

int zx_attn_bwd_noalloc(const void* q, const void* k, const void* v, const void* o, const void* d_o, const float* lse,
                        float* dq, float* dk, float* dv, int B, int Hq, int Hkv, int Sq, int Skv,
                        long long q_tok_stride, long long k_tok_stride, long long v_tok_stride, float scale, int causal,
                        int* status_out, void* stream, char* err, int err_len);

#ifdef __cplusplus
}
#endif
