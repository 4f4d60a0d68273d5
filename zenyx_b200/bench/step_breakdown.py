"""Device time of one full-size micro-batch (8B shape, one 32K sequence), per kind of kernel call.

    python -m zenyx_b200.bench.step_breakdown [--layers 32]

Every GEMM, attention and fused-op call of ``LlamaModel.forward_backward`` is bracketed with CUDA
events on the launching stream; after a warm-up micro-batch the second one is reported, sorted by
share. The event pairs add a few microseconds per call (about 1,500 calls per micro-batch).
"""
from __future__ import annotations

import argparse
import collections

import torch


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--seq-len", type=int, default=32768)
    args = ap.parse_args(argv)
    import zenyx_b200.models.llama as L
    from zenyx_b200.models import LlamaConfig
    from zenyx_b200.models.llama import LlamaModel, RematPolicy

    recs = collections.defaultdict(list)

    def wrap(mod, name, label=None):
        f = getattr(mod, name)

        def g(*a, **k):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            r = f(*a, **k)
            e1.record()
            key = label or name
            if key == "gemm":
                key = f"gemm {tuple(a[0].shape)}x{tuple(a[1].shape)} ta={k.get('trans_a', False)} tb={k.get('trans_b', False)}"
            recs[key].append((e0, e1))
            return r

        setattr(mod, name, g)

    wrap(L, "gemm", "gemm")
    wrap(L, "ring_attn_forward")
    wrap(L, "ring_attn_backward")
    for n in ["rmsnorm_fwd", "rmsnorm_bwd", "rope_qkv_", "rope_bwd_pack", "swiglu_fwd", "swiglu_bwd", "embedding_fwd",
              "embedding_bwd", "cross_entropy_fwd_bwd_"]:
        wrap(L.fused, n)
    cfg = LlamaConfig.llama3_8b()
    cfg.n_layers = args.layers
    model = LlamaModel(cfg, device="cuda", remat=RematPolicy.selective())
    tok = torch.randint(0, cfg.vocab_size, (1, args.seq_len), device="cuda")
    for _ in range(2):
        recs.clear()
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s0.record()
        loss = model.forward_backward(tok, tok)
        s1.record()
        torch.cuda.synchronize()
    tot = s0.elapsed_time(s1)
    print(f"layers {args.layers}: micro-batch device time {tot:.1f} ms, loss {float(loss):.4f}")
    rows = sorted(((sum(a.elapsed_time(b) for a, b in v), k, len(v)) for k, v in recs.items()), reverse=True)
    for ms, k, n in rows:
        print(f"{ms:9.1f} ms  {100 * ms / tot:5.1f}%  n={n:4d}  avg {ms / n:7.3f}  {k}")


if __name__ == "__main__":
    main()
