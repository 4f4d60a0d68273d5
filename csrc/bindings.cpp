// Python bindings of the sm_100a kernels. Tensors are validated here; the kernels themselves see
// raw pointers, the current CUDA stream and one process-wide Status word.
#include <torch/extension.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include "attn/attn.h"
#include "common/status.h"
#include "fused/fused_ops.h"
#include "gemm/gemm.h"
#include "optim/zero.h"
#include "peer/peer.h"

namespace {

using torch::Tensor;

zx::Status* g_status[64] = {nullptr};

zx::Status* status_ptr() {
  int dev = 0;
  cudaGetDevice(&dev);
  if (g_status[dev] == nullptr) {
    zx::Status* p = nullptr;
    TORCH_CHECK(cudaMalloc(&p, sizeof(zx::Status)) == cudaSuccess, "cannot allocate the status word");
    TORCH_CHECK(cudaMemset(p, 0, sizeof(zx::Status)) == cudaSuccess, "cannot clear the status word");
    g_status[dev] = p;
  }
  return g_status[dev];
}

int sm_count() {
  static int n[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (n[dev] == 0) n[dev] = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  return n[dev];
}

cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

void check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  TORCH_CHECK(e == cudaSuccess, what, ": launch failed: ", cudaGetErrorString(e));
}

void check_bf16(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
  TORCH_CHECK(t.scalar_type() == torch::kBFloat16, name, " must be bf16");
}

// Reads (and clears) the device status word. Synchronises the current stream.
std::vector<int64_t> read_status(bool clear) {
  zx::Status h;
  zx::Status* d = status_ptr();
  cudaStream_t st = cur_stream();
  TORCH_CHECK(cudaMemcpyAsync(&h, d, sizeof(h), cudaMemcpyDeviceToHost, st) == cudaSuccess, "status copy failed");
  TORCH_CHECK(cudaStreamSynchronize(st) == cudaSuccess, "stream sync failed while reading the status word");
  if (clear && h.code != 0) cudaMemsetAsync(d, 0, sizeof(h), st);
  return {h.code, h.site, h.block, h.info};
}

// out[M,N] = a @ b^T (+ addend) with optional transposed storage of either operand.
//   a: [M,K] (a_t=false) or [K,M] (a_t=true); b: [N,K] (b_t=false) or [K,N] (b_t=true)
void gemm(const Tensor& a, const Tensor& b, Tensor& out, bool a_t, bool b_t, const c10::optional<Tensor>& addend,
          int64_t pull_src, int64_t pull_dst, int64_t pull_bytes, const std::vector<int64_t>& scatter_ptrs,
          int64_t scatter_rows_per_rank, int64_t scatter_src_rank) {
  check_bf16(a, "a");
  check_bf16(b, "b");
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && out.dim() == 2, "gemm expects matrices");
  TORCH_CHECK(a.stride(1) == 1 && b.stride(1) == 1 && out.stride(1) == 1, "gemm operands must be row-major");
  TORCH_CHECK(out.is_cuda() && (out.scalar_type() == torch::kBFloat16 || out.scalar_type() == torch::kFloat32),
              "out must be bf16 or fp32 on CUDA");
  c10::cuda::CUDAGuard guard(a.device());
  zx::GemmArgs g;
  g.M = (int)(a_t ? a.size(1) : a.size(0));
  g.K = (int)(a_t ? a.size(0) : a.size(1));
  g.N = (int)(b_t ? b.size(1) : b.size(0));
  const int64_t kb = b_t ? b.size(0) : b.size(1);
  TORCH_CHECK(kb == g.K, "gemm: inner dimensions differ (", g.K, " vs ", kb, ")");
  if (scatter_ptrs.empty()) {
    TORCH_CHECK(out.size(0) == g.M && out.size(1) == g.N, "gemm: out has the wrong shape");
  } else {  // `out` is one receive slot of this rank: one rank's rows of the result, bf16
    TORCH_CHECK(out.scalar_type() == torch::kBFloat16 && out.size(0) == scatter_rows_per_rank && out.size(1) == g.N,
                "gemm: a scattered result needs a bf16 [rows_per_rank, N] slot");
  }
  g.A = a.data_ptr();
  g.B = b.data_ptr();
  g.C = out.data_ptr();
  g.lda = (int)a.stride(0);
  g.ldb = (int)b.stride(0);
  g.ldc = (int)out.stride(0);
  g.a_mn = a_t;
  g.b_mn = b_t;
  g.out_fp32 = out.scalar_type() == torch::kFloat32;
  if (addend.has_value()) {
    const Tensor& d = *addend;
    TORCH_CHECK(d.is_cuda() && d.dim() == 2 && d.size(0) == g.M && d.size(1) == g.N && d.stride(1) == 1,
                "gemm: addend must match out");
    TORCH_CHECK(d.scalar_type() == torch::kBFloat16 || d.scalar_type() == torch::kFloat32, "addend must be bf16/fp32");
    g.D = d.data_ptr();
    g.ldd = (int)d.stride(0);
    g.d_mode = d.scalar_type() == torch::kFloat32 ? 2 : 1;
  }
  g.pull_src = reinterpret_cast<const void*>(pull_src);
  g.pull_dst = reinterpret_cast<void*>(pull_dst);
  g.pull_bytes = (size_t)pull_bytes;
  if (!scatter_ptrs.empty()) {
    TORCH_CHECK(scatter_ptrs.size() <= 8 && scatter_rows_per_rank > 0, "gemm: at most 8 scatter targets");
    TORCH_CHECK(!addend.has_value(), "gemm: a scattered result takes no addend");
    g.scatter_ranks = (int)scatter_ptrs.size();
    g.scatter_rows_per_rank = (int)scatter_rows_per_rank;
    g.scatter_src_rank = (int)scatter_src_rank;
    for (size_t r = 0; r < scatter_ptrs.size(); ++r) g.scatter_base[r] = reinterpret_cast<void*>(scatter_ptrs[r]);
  }
  g.status = status_ptr();
  g.stream = cur_stream();
  g.sm_count = sm_count();
  zx::launch_gemm_bf16(g);
  check_launch("gemm");
}

zx::AttnLayout to_layout(const std::vector<int64_t>& pos, int64_t S) {
  zx::AttnLayout l;
  TORCH_CHECK(!pos.empty() && (int)pos.size() <= zx::kAttnMaxChunks, "between 1 and 8 chunks are supported");
  l.n_chunks = (int)pos.size();
  TORCH_CHECK(S % l.n_chunks == 0, "the buffer must split evenly into its chunks");
  l.chunk_len = (int)(S / l.n_chunks);
  for (int i = 0; i < l.n_chunks; ++i) l.chunk_pos[i] = (int)pos[i];
  return l;
}

void check_qkv(const Tensor& t, const char* name) {
  check_bf16(t, name);
  TORCH_CHECK(t.dim() == 4 && t.size(3) == 128, name, " must be [B, S, H, 128]");
  TORCH_CHECK(t.stride(3) == 1 && t.stride(2) == 128, name, ": heads must be contiguous 128-vectors");
  TORCH_CHECK(t.stride(0) == t.size(1) * t.stride(1), name, ": batch stride must equal S * token stride");
  TORCH_CHECK(t.stride(1) % 8 == 0, name, ": token stride must keep 16-byte alignment");
}

// q [B,Sq,Hq,128], k/v [B,Skv,Hkv,128] (token-strided views are fine); o [B,Sq,Hq,128], lse [B,Hq,Sq].
void attn_fwd(const Tensor& q, const Tensor& k, const Tensor& v, Tensor& o, Tensor& lse, double scale, bool causal,
              int64_t window_blocks, int64_t global_every, const std::vector<int64_t>& q_chunk_pos,
              const std::vector<int64_t>& kv_chunk_pos, bool merge_prev, int64_t pull_src, int64_t pull_dst,
              int64_t pull_bytes) {
  check_qkv(q, "q");
  check_qkv(k, "k");
  check_qkv(v, "v");
  check_bf16(o, "o");
  TORCH_CHECK(o.is_contiguous() && o.sizes() == q.sizes(), "o must be contiguous with q's shape");
  TORCH_CHECK(lse.is_cuda() && lse.scalar_type() == torch::kFloat32 && lse.is_contiguous(), "lse must be fp32");
  TORCH_CHECK(lse.dim() == 3 && lse.size(0) == q.size(0) && lse.size(1) == q.size(2) && lse.size(2) == q.size(1),
              "lse must be [B, Hq, Sq]");
  TORCH_CHECK(k.sizes() == v.sizes() && k.size(0) == q.size(0), "k and v must agree");
  c10::cuda::CUDAGuard guard(q.device());
  zx::AttnFwdArgs a;
  a.q = q.data_ptr(); a.k = k.data_ptr(); a.v = v.data_ptr(); a.o = o.data_ptr();
  a.lse = lse.data_ptr<float>();
  a.B = (int)q.size(0); a.Sq = (int)q.size(1); a.Hq = (int)q.size(2);
  a.Skv = (int)k.size(1); a.Hkv = (int)k.size(2);
  a.q_tok_stride = q.stride(1); a.k_tok_stride = k.stride(1); a.v_tok_stride = v.stride(1);
  a.scale = (float)scale;
  a.mask.causal = causal; a.mask.window_blocks = (int)window_blocks; a.mask.global_every = (int)global_every;
  a.q_layout = to_layout(q_chunk_pos, a.Sq);
  a.kv_layout = to_layout(kv_chunk_pos, a.Skv);
  a.merge_prev = merge_prev;
  a.pull_src = reinterpret_cast<const void*>(pull_src);
  a.pull_dst = reinterpret_cast<void*>(pull_dst);
  a.pull_bytes = (size_t)pull_bytes;
  a.status = status_ptr();
  a.stream = cur_stream();
  zx::launch_attn_fwd(a);
  check_launch("attn_fwd");
}

void attn_bwd(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& o, const Tensor& d_o, const Tensor& lse,
              Tensor& delta, Tensor& dq, Tensor& dk, Tensor& dv, double scale, bool causal, int64_t window_blocks,
              int64_t global_every, const std::vector<int64_t>& q_chunk_pos, const std::vector<int64_t>& kv_chunk_pos,
              bool compute_delta, bool dq_accumulate, int64_t pull_src, int64_t pull_dst, int64_t pull_bytes,
              const c10::optional<Tensor>& trace) {
  check_qkv(q, "q");
  check_qkv(k, "k");
  check_qkv(v, "v");
  check_bf16(o, "o");
  check_bf16(d_o, "d_o");
  TORCH_CHECK(o.is_contiguous() && d_o.is_contiguous() && o.sizes() == q.sizes() && d_o.sizes() == q.sizes(),
              "o and d_o must be contiguous with q's shape");
  for (const Tensor* t : std::initializer_list<const Tensor*>{&lse, &delta, &dq, &dk, &dv})
    TORCH_CHECK(t->is_cuda() && t->scalar_type() == torch::kFloat32 && t->is_contiguous(), "fp32 contiguous expected");
  TORCH_CHECK(dq.sizes() == q.sizes() && dk.sizes() == k.sizes() && dv.sizes() == v.sizes(), "gradient shapes differ");
  TORCH_CHECK(delta.sizes() == lse.sizes(), "delta must match lse");
  c10::cuda::CUDAGuard guard(q.device());
  zx::AttnBwdArgs a;
  a.q = q.data_ptr(); a.k = k.data_ptr(); a.v = v.data_ptr(); a.o = o.data_ptr(); a.d_o = d_o.data_ptr();
  a.lse = lse.data_ptr<float>(); a.delta = delta.data_ptr<float>();
  a.dq = dq.data_ptr<float>(); a.dk = dk.data_ptr<float>(); a.dv = dv.data_ptr<float>();
  a.B = (int)q.size(0); a.Sq = (int)q.size(1); a.Hq = (int)q.size(2);
  a.Skv = (int)k.size(1); a.Hkv = (int)k.size(2);
  a.q_tok_stride = q.stride(1); a.k_tok_stride = k.stride(1); a.v_tok_stride = v.stride(1);
  a.scale = (float)scale;
  a.mask.causal = causal; a.mask.window_blocks = (int)window_blocks; a.mask.global_every = (int)global_every;
  a.q_layout = to_layout(q_chunk_pos, a.Sq);
  a.kv_layout = to_layout(kv_chunk_pos, a.Skv);
  a.compute_delta = compute_delta;
  a.dq_accumulate = dq_accumulate;
  a.pull_src = reinterpret_cast<const void*>(pull_src);
  a.pull_dst = reinterpret_cast<void*>(pull_dst);
  a.pull_bytes = (size_t)pull_bytes;
  if (trace.has_value()) {
    TORCH_CHECK(trace->is_cuda() && trace->scalar_type() == torch::kInt64 && trace->numel() >= 3072, "trace: int64[3072]");
    a.trace = reinterpret_cast<long long*>(trace->data_ptr());
  }
  a.status = status_ptr();
  a.stream = cur_stream();
  zx::launch_attn_bwd(a);
  check_launch("attn_bwd");
}

void rmsnorm_fwd(const Tensor& x, const Tensor& w, Tensor& y, Tensor& rstd, double eps) {
  check_bf16(x, "x"); check_bf16(w, "w"); check_bf16(y, "y");
  TORCH_CHECK(x.is_contiguous() && y.is_contiguous() && w.is_contiguous(), "rmsnorm: contiguous tensors expected");
  const int H = (int)x.size(-1);
  TORCH_CHECK(H % 8 == 0 && w.numel() == H, "rmsnorm: hidden size must be a multiple of 8");
  const int rows = (int)(x.numel() / H);
  TORCH_CHECK(rstd.scalar_type() == torch::kFloat32 && rstd.numel() == rows, "rstd must be fp32 [rows]");
  c10::cuda::CUDAGuard guard(x.device());
  zx::launch_rmsnorm_fwd(x.data_ptr(), w.data_ptr(), y.data_ptr(), rstd.data_ptr<float>(), rows, H, (float)eps,
                         cur_stream());
  check_launch("rmsnorm_fwd");
}

void rmsnorm_bwd(const Tensor& dy, const Tensor& x, const Tensor& w, const Tensor& rstd, Tensor& dx, Tensor& dw_accum,
                 const c10::optional<Tensor>& dres) {
  check_bf16(dy, "dy"); check_bf16(x, "x"); check_bf16(w, "w"); check_bf16(dx, "dx");
  TORCH_CHECK(dy.is_contiguous() && x.is_contiguous() && dx.is_contiguous(), "rmsnorm_bwd: contiguous expected");
  const int H = (int)x.size(-1);
  const int rows = (int)(x.numel() / H);
  TORCH_CHECK(dw_accum.scalar_type() == torch::kFloat32 && dw_accum.numel() == H && dw_accum.is_contiguous(),
              "dw_accum must be fp32 [H]");
  TORCH_CHECK((size_t)H * 4 <= 48 * 1024, "rmsnorm_bwd: hidden size too large for the shared accumulator");
  c10::cuda::CUDAGuard guard(x.device());
  const void* dres_p = nullptr;
  if (dres.has_value()) {
    check_bf16(*dres, "dres");
    TORCH_CHECK(dres->is_contiguous() && dres->numel() == x.numel(), "dres must match x");
    dres_p = dres->data_ptr();
  }
  zx::launch_rmsnorm_bwd(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr<float>(), dres_p, dx.data_ptr(),
                         dw_accum.data_ptr<float>(), rows, H, sm_count(), cur_stream());
  check_launch("rmsnorm_bwd");
}

// qkv: [tokens, (Hq + 2 Hkv) * D] rotated in place (Q, and K unless k_out is given).
void rope_qkv(Tensor& qkv, const Tensor& cos_t, const Tensor& sin_t, const c10::optional<Tensor>& k_out,
              const c10::optional<Tensor>& v_out, int64_t Hq, int64_t Hkv, int64_t D, int64_t tokens_per_seq,
              bool inverse) {
  check_bf16(qkv, "qkv");
  TORCH_CHECK(qkv.is_contiguous() && qkv.dim() == 2 && qkv.size(1) == (Hq + 2 * Hkv) * D, "qkv has the wrong shape");
  TORCH_CHECK(D % 16 == 0, "rope: head_dim must be a multiple of 16");
  TORCH_CHECK(cos_t.scalar_type() == torch::kFloat32 && sin_t.scalar_type() == torch::kFloat32 &&
                  cos_t.is_contiguous() && sin_t.is_contiguous() && cos_t.size(0) >= tokens_per_seq &&
                  cos_t.size(1) == D / 2 && sin_t.sizes() == cos_t.sizes(),
              "rope tables must be fp32 [tokens_per_seq, D/2]");
  void* kp = nullptr;
  void* vp = nullptr;
  if (k_out.has_value()) {
    check_bf16(*k_out, "k_out");
    TORCH_CHECK(k_out->is_contiguous() && k_out->numel() == qkv.size(0) * Hkv * D, "k_out has the wrong size");
    kp = k_out->data_ptr();
  }
  if (v_out.has_value()) {
    check_bf16(*v_out, "v_out");
    TORCH_CHECK(v_out->is_contiguous() && v_out->numel() == qkv.size(0) * Hkv * D, "v_out has the wrong size");
    vp = v_out->data_ptr();
  }
  c10::cuda::CUDAGuard guard(qkv.device());
  zx::launch_rope_qkv(qkv.data_ptr(), cos_t.data_ptr<float>(), sin_t.data_ptr<float>(), kp, vp, (int)qkv.size(0),
                      (int)tokens_per_seq, (int)Hq, (int)Hkv, (int)D, inverse ? -1.f : 1.f, sm_count(), cur_stream());
  check_launch("rope_qkv");
}

// fp32 dq [T,Hq,D], dk/dv [T,Hkv,D] -> bf16 dqkv [T,(Hq+2Hkv)*D] with the inverse rotation on dq, dk
void rope_bwd_pack(const Tensor& dq, const Tensor& dk, const Tensor& dv, const Tensor& cos_t, const Tensor& sin_t,
                   Tensor& dqkv, int64_t Hq, int64_t Hkv, int64_t D, int64_t tokens_per_seq) {
  check_bf16(dqkv, "dqkv");
  for (const Tensor* t : std::initializer_list<const Tensor*>{&dq, &dk, &dv, &cos_t, &sin_t})
    TORCH_CHECK(t->is_cuda() && t->scalar_type() == torch::kFloat32 && t->is_contiguous(), "fp32 contiguous expected");
  const int64_t T = dqkv.size(0);
  TORCH_CHECK(dqkv.is_contiguous() && dqkv.size(1) == (Hq + 2 * Hkv) * D && D % 16 == 0, "dqkv shape");
  TORCH_CHECK(dq.numel() == T * Hq * D && dk.numel() == T * Hkv * D && dv.numel() == T * Hkv * D, "gradient sizes");
  TORCH_CHECK(cos_t.size(0) >= tokens_per_seq && cos_t.size(1) == D / 2, "rope tables");
  c10::cuda::CUDAGuard guard(dqkv.device());
  zx::launch_rope_bwd_pack(dq.data_ptr<float>(), dk.data_ptr<float>(), dv.data_ptr<float>(), cos_t.data_ptr<float>(),
                           sin_t.data_ptr<float>(), dqkv.data_ptr(), (int)T, (int)tokens_per_seq, (int)Hq, (int)Hkv,
                           (int)D, sm_count(), cur_stream());
  check_launch("rope_bwd_pack");
}

void swiglu_fwd(const Tensor& gu, Tensor& h) {
  check_bf16(gu, "gu"); check_bf16(h, "h");
  TORCH_CHECK(gu.is_contiguous() && h.is_contiguous() && gu.dim() == 2 && gu.size(1) == 2 * h.size(1) &&
                  gu.size(0) == h.size(0) && h.size(1) % 8 == 0, "swiglu shapes");
  c10::cuda::CUDAGuard guard(gu.device());
  zx::launch_swiglu_fwd(gu.data_ptr(), h.data_ptr(), (size_t)h.size(0), (int)h.size(1), sm_count(), cur_stream());
  check_launch("swiglu_fwd");
}
void swiglu_bwd(const Tensor& gu, const Tensor& dh, Tensor& dgu) {
  check_bf16(gu, "gu"); check_bf16(dh, "dh"); check_bf16(dgu, "dgu");
  TORCH_CHECK(gu.is_contiguous() && dh.is_contiguous() && dgu.is_contiguous() && dgu.sizes() == gu.sizes() &&
                  gu.size(1) == 2 * dh.size(1) && dh.size(1) % 8 == 0, "swiglu_bwd shapes");
  c10::cuda::CUDAGuard guard(gu.device());
  zx::launch_swiglu_bwd(gu.data_ptr(), dh.data_ptr(), dgu.data_ptr(), (size_t)dh.size(0), (int)dh.size(1), sm_count(),
                        cur_stream());
  check_launch("swiglu_bwd");
}

void embedding_fwd(const Tensor& ids, const Tensor& table, Tensor& out) {
  check_bf16(table, "table"); check_bf16(out, "out");
  TORCH_CHECK(ids.is_cuda() && ids.scalar_type() == torch::kInt64 && ids.is_contiguous(), "ids must be int64");
  TORCH_CHECK(table.is_contiguous() && out.is_contiguous() && out.numel() == ids.numel() * table.size(1), "shapes");
  c10::cuda::CUDAGuard guard(table.device());
  zx::launch_embedding_fwd(ids.data_ptr<int64_t>(), table.data_ptr(), out.data_ptr(), (size_t)ids.numel(),
                           (int)table.size(1), (int)table.size(0), sm_count(), cur_stream());
  check_launch("embedding_fwd");
}
void embedding_bwd(const Tensor& ids, const Tensor& dout, Tensor& dtable) {
  check_bf16(dout, "dout");
  TORCH_CHECK(ids.is_cuda() && ids.scalar_type() == torch::kInt64 && ids.is_contiguous(), "ids must be int64");
  TORCH_CHECK(dtable.scalar_type() == torch::kFloat32 && dtable.is_contiguous() && dout.is_contiguous() &&
                  dout.numel() == ids.numel() * dtable.size(1), "shapes");
  c10::cuda::CUDAGuard guard(dout.device());
  zx::launch_embedding_bwd(ids.data_ptr<int64_t>(), dout.data_ptr(), dtable.data_ptr<float>(), (size_t)ids.numel(),
                           (int)dtable.size(1), (int)dtable.size(0), sm_count(), cur_stream());
  check_launch("embedding_bwd");
}

// logits [rows, V] are replaced by d(loss_sum)/d(logits) * grad_scale; loss [rows] gets the per-token loss.
void ce_fwd_bwd(Tensor& logits, const Tensor& targets, Tensor& loss, double grad_scale, int64_t ignore_index) {
  check_bf16(logits, "logits");
  TORCH_CHECK(logits.dim() == 2 && logits.stride(1) == 1 && logits.size(1) % 8 == 0 && logits.stride(0) % 8 == 0,
              "logits must be [rows, V] with V a multiple of 8");
  TORCH_CHECK(targets.is_cuda() && targets.scalar_type() == torch::kInt64 && targets.is_contiguous() &&
                  targets.numel() == logits.size(0), "targets must be int64 [rows]");
  TORCH_CHECK(loss.scalar_type() == torch::kFloat32 && loss.is_contiguous() && loss.numel() == logits.size(0),
              "loss must be fp32 [rows]");
  c10::cuda::CUDAGuard guard(logits.device());
  zx::launch_ce_fwd_bwd(logits.data_ptr(), targets.data_ptr<int64_t>(), loss.data_ptr<float>(), (int)logits.size(0),
                        (int)logits.size(1), (int)logits.stride(0), (float)grad_scale, (int)ignore_index, cur_stream());
  check_launch("ce_fwd_bwd");
}

// x [tokens, Hkv, D] -> q uint8 (e4m3 bits) + scales [ceil(tokens/block), Hkv] (+ power-of-two scales)
void kv_quant_e4m3(const Tensor& x, Tensor& q, Tensor& scales, const c10::optional<Tensor>& scales_pow2,
                   int64_t block_tokens) {
  check_bf16(x, "x");
  TORCH_CHECK(x.dim() == 3 && x.is_contiguous() && x.size(2) % 8 == 0, "x must be [tokens, Hkv, D]");
  TORCH_CHECK(q.is_cuda() && q.element_size() == 1 && q.is_contiguous() && q.numel() == x.numel(), "q must be 1-byte");
  const int64_t blocks = (x.size(0) + block_tokens - 1) / block_tokens;
  TORCH_CHECK(scales.scalar_type() == torch::kFloat32 && scales.is_contiguous() && scales.numel() == blocks * x.size(1),
              "scales must be fp32 [blocks, Hkv]");
  float* sp2 = nullptr;
  if (scales_pow2.has_value()) {
    TORCH_CHECK(scales_pow2->scalar_type() == torch::kFloat32 && scales_pow2->numel() == scales.numel(), "pow2 scales");
    sp2 = scales_pow2->data_ptr<float>();
  }
  c10::cuda::CUDAGuard guard(x.device());
  zx::launch_kv_quant_e4m3(x.data_ptr(), q.data_ptr(), scales.data_ptr<float>(), sp2, (int)x.size(0), (int)x.size(1),
                           (int)x.size(2), (int)block_tokens, cur_stream());
  check_launch("kv_quant_e4m3");
}
void kv_dequant_e4m3(const Tensor& q, const Tensor& scales, Tensor& x, int64_t block_tokens) {
  check_bf16(x, "x");
  TORCH_CHECK(x.dim() == 3 && x.is_contiguous() && q.is_contiguous() && q.numel() == x.numel(), "shapes");
  c10::cuda::CUDAGuard guard(x.device());
  zx::launch_kv_dequant_e4m3(q.data_ptr(), scales.data_ptr<float>(), x.data_ptr(), (size_t)x.size(0), (int)x.size(1),
                             (int)x.size(2), (int)block_tokens, sm_count(), cur_stream());
  check_launch("kv_dequant_e4m3");
}

// AdamW over flat buffers of n (multiple of 4) elements; see fused_ops.cu for the master split.
void adamw(Tensor& p_hi, Tensor& p_lo, Tensor& m, Tensor& v, const Tensor& g, double lr, double beta1, double beta2,
           double eps, double weight_decay, int64_t step, double grad_scale, const c10::optional<Tensor>& scale_ptr) {
  const int64_t n = g.numel();
  TORCH_CHECK(n % 4 == 0, "adamw: element count must be a multiple of 4");
  TORCH_CHECK(p_hi.is_cuda() && p_hi.element_size() == 2 && p_lo.element_size() == 2 && p_hi.numel() == n &&
                  p_lo.numel() == n && m.numel() == n && v.numel() == n, "adamw: size mismatch");
  TORCH_CHECK(m.scalar_type() == torch::kFloat32 && v.scalar_type() == torch::kFloat32 &&
                  g.scalar_type() == torch::kFloat32, "adamw: m, v, g must be fp32");
  TORCH_CHECK(p_hi.is_contiguous() && p_lo.is_contiguous() && m.is_contiguous() && v.is_contiguous() && g.is_contiguous(),
              "adamw: contiguous buffers expected");
  const float* sp = nullptr;
  if (scale_ptr.has_value()) sp = scale_ptr->data_ptr<float>();
  c10::cuda::CUDAGuard guard(g.device());
  zx::launch_adamw(p_hi.data_ptr(), p_lo.data_ptr(), m.data_ptr<float>(), v.data_ptr<float>(), g.data_ptr<float>(),
                   (size_t)n, (float)lr, (float)beta1, (float)beta2, (float)eps, (float)weight_decay, (int)step,
                   (float)grad_scale, sp, sm_count(), cur_stream());
  check_launch("adamw");
}

void sumsq(const Tensor& g, Tensor& out) {
  TORCH_CHECK(g.is_cuda() && g.scalar_type() == torch::kFloat32 && g.is_contiguous() && g.numel() % 4 == 0, "sumsq: g");
  TORCH_CHECK(out.scalar_type() == torch::kFloat32 && out.numel() >= 1, "sumsq: out");
  c10::cuda::CUDAGuard guard(g.device());
  zx::launch_sumsq(g.data_ptr<float>(), (size_t)g.numel(), out.data_ptr<float>(), sm_count(), cur_stream());
  check_launch("sumsq");
}
void sum_slots_bf16(const Tensor& slots, int64_t ranks, Tensor& out) {
  TORCH_CHECK(slots.is_cuda() && slots.scalar_type() == torch::kBFloat16 && slots.is_contiguous(), "sum_slots: slots");
  TORCH_CHECK(out.is_cuda() && out.scalar_type() == torch::kBFloat16 && out.is_contiguous() && out.numel() % 8 == 0 &&
                  slots.numel() == ranks * out.numel(),
              "sum_slots: out must be contiguous bf16 with numel a multiple of 8 and slots = ranks x out");
  c10::cuda::CUDAGuard guard(out.device());
  zx::launch_sum_slots_bf16(slots.data_ptr(), (int)ranks, (size_t)out.numel(), out.data_ptr(), sm_count(), cur_stream());
  check_launch("sum_slots_bf16");
}
void clip_coef(const Tensor& ss, double scale, double max_norm, Tensor& coef, Tensor& norm_out) {
  c10::cuda::CUDAGuard guard(ss.device());
  zx::launch_clip_coef(ss.data_ptr<float>(), (float)scale, (float)max_norm, coef.data_ptr<float>(),
                       norm_out.data_ptr<float>(), cur_stream());
  check_launch("clip_coef");
}

// ---------------------------------------------------------------------------------------------
// Peer memory and the fused optimizer
// ---------------------------------------------------------------------------------------------
int64_t peer_alloc(int64_t bytes) { return reinterpret_cast<int64_t>(zx::peer_alloc((size_t)bytes)); }
py::bytes peer_export(int64_t ptr) { return py::bytes(zx::peer_export(reinterpret_cast<void*>(ptr))); }
int64_t peer_open(const std::string& handle) { return reinterpret_cast<int64_t>(zx::peer_open(handle)); }
void peer_close(int64_t ptr) { zx::peer_close(reinterpret_cast<void*>(ptr)); }
void peer_free(int64_t ptr) { zx::peer_free(reinterpret_cast<void*>(ptr)); }

// A tensor view over raw device memory (own or peer-mapped). The caller keeps the memory alive.
Tensor tensor_from_ptr(int64_t ptr, const std::vector<int64_t>& sizes, torch::ScalarType dtype) {
  int dev = 0;
  cudaGetDevice(&dev);
  auto opts = torch::TensorOptions().dtype(dtype).device(torch::kCUDA, dev);
  return torch::from_blob(reinterpret_cast<void*>(ptr), sizes, [](void*) {}, opts);
}

zx::PeerPtrs to_ptrs(const std::vector<int64_t>& v) {
  TORCH_CHECK(!v.empty() && (int)v.size() <= zx::kMaxPeers, "between 1 and 8 peers are supported");
  zx::PeerPtrs p;
  for (int i = 0; i < zx::kMaxPeers; ++i) p.p[i] = i < (int)v.size() ? reinterpret_cast<void*>(v[i]) : nullptr;
  return p;
}

void peer_barrier(const std::vector<int64_t>& flag_ptrs, int64_t rank, int64_t epoch, double timeout_ms) {
  zx::launch_peer_barrier(to_ptrs(flag_ptrs), (int)rank, (int)flag_ptrs.size(), (uint32_t)epoch,
                          (uint64_t)(timeout_ms * 1e6), status_ptr(), cur_stream());
  check_launch("peer_barrier");
}

void peer_pull(int64_t src_ptr, int64_t dst_ptr, int64_t bytes, int64_t blocks) {
  TORCH_CHECK(bytes % 16 == 0, "peer_pull: size must be a multiple of 16 bytes");
  zx::launch_peer_pull(reinterpret_cast<const void*>(src_ptr), reinterpret_cast<void*>(dst_ptr), (size_t)bytes,
                       (int)blocks, cur_stream());
  check_launch("peer_pull");
}

void zero_step(const std::vector<int64_t>& grad_ptrs, const std::vector<int64_t>& param_ptrs, int64_t rank,
               int64_t shard_begin, int64_t n_shard, int64_t decay_end, const c10::optional<Tensor>& g_shard,
               Tensor& p_lo, Tensor& m, Tensor& v, const c10::optional<Tensor>& sumsq,
               const c10::optional<Tensor>& clip_coef, bool do_reduce, bool do_update, bool zero_grads,
               double grad_scale, double lr, double beta1, double beta2, double eps, double weight_decay,
               int64_t step) {
  TORCH_CHECK(grad_ptrs.size() == param_ptrs.size(), "zero_step: peer lists differ");
  TORCH_CHECK(shard_begin % 4 == 0 && n_shard % 4 == 0, "zero_step: shard bounds must be multiples of 4");
  TORCH_CHECK(p_lo.is_cuda() && p_lo.element_size() == 2 && p_lo.numel() >= n_shard && m.numel() >= n_shard &&
                  v.numel() >= n_shard && m.scalar_type() == v.scalar_type() &&
                  (m.scalar_type() == torch::kFloat32 || m.scalar_type() == torch::kBFloat16) && m.is_contiguous() &&
                  v.is_contiguous(),
              "zero_step: shard state has the wrong size or type");
  zx::ZeroArgs a;
  a.grads = to_ptrs(grad_ptrs);
  a.params = to_ptrs(param_ptrs);
  a.nranks = (int)grad_ptrs.size();
  a.rank = (int)rank;
  a.shard_begin = (size_t)shard_begin;
  a.n_shard = (size_t)n_shard;
  a.decay_end = (size_t)decay_end;
  if (g_shard.has_value()) {
    TORCH_CHECK(g_shard->scalar_type() == torch::kFloat32 && g_shard->numel() >= n_shard, "zero_step: g_shard");
    a.g_shard = g_shard->data_ptr<float>();
  } else {
    // without a shard buffer a pass either updates straight from the reduced gradients, or (norm pass)
    // only accumulates their sum of squares and leaves them in place for a second reducing pass
    TORCH_CHECK(do_reduce && (do_update || !zero_grads), "zero_step: this pass needs a g_shard buffer");
  }
  a.p_lo = reinterpret_cast<int16_t*>(p_lo.data_ptr());
  a.m = m.data_ptr();
  a.v = v.data_ptr();
  a.state_bf16 = m.scalar_type() == torch::kBFloat16 ? 1 : 0;
  a.sumsq = sumsq.has_value() ? sumsq->data_ptr<float>() : nullptr;
  a.clip_coef = clip_coef.has_value() ? clip_coef->data_ptr<float>() : nullptr;
  a.do_reduce = do_reduce; a.do_update = do_update; a.zero_grads = zero_grads;
  a.grad_scale = (float)grad_scale; a.lr = (float)lr; a.beta1 = (float)beta1; a.beta2 = (float)beta2;
  a.eps = (float)eps; a.weight_decay = (float)weight_decay; a.step = (int)step;
  a.sm_count = sm_count();
  a.stream = cur_stream();
  c10::cuda::CUDAGuard guard(m.device());
  zx::launch_zero_step(a);
  check_launch("zero_step");
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("read_status", &read_status, "read (and optionally clear) the kernel status word");
  m.def("gemm", &gemm, py::arg("a"), py::arg("b"), py::arg("out"), py::arg("a_t"), py::arg("b_t"), py::arg("addend"),
        py::arg("pull_src") = 0, py::arg("pull_dst") = 0, py::arg("pull_bytes") = 0,
        py::arg("scatter_ptrs") = std::vector<int64_t>{}, py::arg("scatter_rows_per_rank") = 0, py::arg("scatter_src_rank") = 0);
  m.def("attn_fwd", &attn_fwd);
  m.def("attn_bwd", &attn_bwd, py::arg("q"), py::arg("k"), py::arg("v"), py::arg("o"), py::arg("d_o"), py::arg("lse"),
        py::arg("delta"), py::arg("dq"), py::arg("dk"), py::arg("dv"), py::arg("scale"), py::arg("causal"),
        py::arg("window_blocks"), py::arg("global_every"), py::arg("q_chunk_pos"), py::arg("kv_chunk_pos"),
        py::arg("compute_delta"), py::arg("dq_accumulate"), py::arg("pull_src"), py::arg("pull_dst"),
        py::arg("pull_bytes"), py::arg("trace") = py::none());
  m.def("rmsnorm_fwd", &rmsnorm_fwd);
  m.def("rmsnorm_bwd", &rmsnorm_bwd);
  m.def("rope_qkv", &rope_qkv);
  m.def("rope_bwd_pack", &rope_bwd_pack);
  m.def("swiglu_fwd", &swiglu_fwd);
  m.def("swiglu_bwd", &swiglu_bwd);
  m.def("embedding_fwd", &embedding_fwd);
  m.def("embedding_bwd", &embedding_bwd);
  m.def("ce_fwd_bwd", &ce_fwd_bwd);
  m.def("kv_quant_e4m3", &kv_quant_e4m3);
  m.def("kv_dequant_e4m3", &kv_dequant_e4m3);
  m.def("adamw", &adamw);
  m.def("sumsq", &sumsq);
  m.def("clip_coef", &clip_coef);
  m.def("sum_slots_bf16", &sum_slots_bf16);
  m.def("peer_alloc", &peer_alloc);
  m.def("peer_export", &peer_export);
  m.def("peer_open", &peer_open);
  m.def("peer_close", &peer_close);
  m.def("peer_free", &peer_free);
  m.def("tensor_from_ptr", &tensor_from_ptr);
  m.def("peer_barrier", &peer_barrier);
  m.def("peer_pull", &peer_pull);
  m.def("zero_step", &zero_step);
}
