"""Multi-GPU worker run under torch.distributed.run by tests/test_gpu_dist.py (one rank per GPU)."""
import math
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


def case_ring(ctx):
    from zenyx_b200.ops import _ext
    from zenyx_b200.ops.attention import (MaskSpec, RingContext, _positions, attn_backward, attn_forward,
                                          ring_attn_backward, ring_attn_forward, shard_sequence)
    from zenyx_b200.parallel.peer import RingBuffers

    R, r = ctx.world_size, ctx.rank
    B, S, Hq, Hkv, D = 1, 512 * R, 4, 2, 128
    g = torch.Generator(device="cuda").manual_seed(5)
    q = torch.randn(B, S, Hq, D, device="cuda", generator=g).bfloat16()
    k = torch.randn(B, S, Hkv, D, device="cuda", generator=g).bfloat16()
    v = torch.randn(B, S, Hkv, D, device="cuda", generator=g).bfloat16()
    do = torch.randn(B, S, Hq, D, device="cuda", generator=g).bfloat16()
    scale = 1 / math.sqrt(D)
    for mask in (MaskSpec(True), MaskSpec(True, 2, 4)):
        # single-GPU result with the same kernels (identical on every rank)
        o_ref = torch.empty_like(q)
        lse_ref = torch.empty(B, Hq, S, device="cuda")
        attn_forward(q, k, v, o_ref, lse_ref, scale, mask, [0], [0])
        dq_ref = torch.empty(B, S, Hq, D, device="cuda")
        dk_ref = torch.zeros(B, S, Hkv, D, device="cuda")
        dv_ref = torch.zeros(B, S, Hkv, D, device="cuda")
        attn_backward(q, k, v, o_ref, do, lse_ref, torch.empty_like(lse_ref), dq_ref, dk_ref, dv_ref, scale, mask, [0], [0])
        peer = RingBuffers((B, S // R, Hkv, D), group=None, timeout_ms=5000.0)
        ring = RingContext(rank=r, degree=R, seq_len=S, peer=peer, mask=mask)
        ql, dol = shard_sequence(q, r, R).contiguous(), shard_sequence(do, r, R).contiguous()
        ks, vs = peer.kv_views(r, 0)
        ks.copy_(shard_sequence(k, r, R))
        vs.copy_(shard_sequence(v, r, R))
        o, lse = ring_attn_forward(ring, ql, ks, vs, scale, 0)
        dq, dk, dv = ring_attn_backward(ring, ql, ks, vs, o, dol, lse, scale, 0)
        _ext.check_status()
        errs = {
            "o": rel(o, shard_sequence(o_ref, r, R)),
            "lse": (lse - shard_sequence(lse_ref, r, R, dim=2)).abs().max().item(),
            "dq": rel(dq, shard_sequence(dq_ref, r, R)),
            "dk": rel(dk, shard_sequence(dk_ref, r, R)),
            "dv": rel(dv, shard_sequence(dv_ref, r, R)),
        }
        assert all(e < 2e-2 for e in errs.values()), (mask, errs)
        # the ring result against fp32 math as well (not only against this package's single-GPU kernels)
        from zenyx_b200.bench.ring_attn import slice_check

        chk = slice_check(ring, ql, ks, vs, dol, o, lse, dq, dk, dv, scale, mask, n_check=S // 2)
        assert chk["ok"] and max(chk[n]["max_abs"] for n in ("o", "dq", "dk", "dv")) < 0.25, chk
        torch.cuda.synchronize()
        dist.barrier()
        peer.close()
    # e4m3 cache format in the peer slots and on the wire: same result as one GPU attending the round-tripped K/V
    from zenyx_b200.train.fp8_kv_quantization import FP8KVQuantizer

    qz = FP8KVQuantizer(Hkv, D, 128)
    kq, vq = qz.roundtrip(k), qz.roundtrip(v)
    mask = MaskSpec(True)
    o_ref = torch.empty_like(q)
    lse_ref = torch.empty(B, Hq, S, device="cuda")
    attn_forward(q, kq, vq, o_ref, lse_ref, scale, mask, [0], [0])
    dq_ref = torch.empty(B, S, Hq, D, device="cuda")
    dk_ref = torch.zeros(B, S, Hkv, D, device="cuda")
    dv_ref = torch.zeros(B, S, Hkv, D, device="cuda")
    attn_backward(q, kq, vq, o_ref, do, lse_ref, torch.empty_like(lse_ref), dq_ref, dk_ref, dv_ref, scale, mask, [0], [0])
    peer = RingBuffers((B, S // R, Hkv, D), group=None, timeout_ms=5000.0, fp8_block_tokens=128)
    ring = RingContext(rank=r, degree=R, seq_len=S, peer=peer, mask=mask)
    ql, dol = shard_sequence(q, r, R).contiguous(), shard_sequence(do, r, R).contiguous()
    kl, vl = shard_sequence(k, r, R).contiguous(), shard_sequence(v, r, R).contiguous()
    o, lse = ring_attn_forward(ring, ql, kl, vl, scale, 0)
    dq, dk, dv = ring_attn_backward(ring, ql, kl, vl, o, dol, lse, scale, 0)
    _ext.check_status()
    errs = {"o": rel(o, shard_sequence(o_ref, r, R)), "dq": rel(dq, shard_sequence(dq_ref, r, R)),
            "dk": rel(dk, shard_sequence(dk_ref, r, R)), "dv": rel(dv, shard_sequence(dv_ref, r, R))}
    assert all(e < 2e-2 for e in errs.values()), ("fp8 ring", errs)
    assert peer.pull_args((r + 1) % R, 0, 0)[2] < 0.55 * 2 * (S // R) * Hkv * D * 2    # about half the bf16 bytes
    torch.cuda.synchronize()
    dist.barrier()
    peer.close()
    print(f"rank {r}: ring ok", flush=True)


def case_zero(ctx):
    from zenyx_b200.models.llama import FlatBuffers
    from zenyx_b200.ops import _ext, fused
    from zenyx_b200.parallel.zero import ZeroAdamW

    R, r = ctx.world_size, ctx.rank
    specs = [("a", (1000, 64), True), ("b", (300, 128), True), ("n", (512,), False)]
    results = {}
    for fused_peer in (True, False):
        flat = FlatBuffers(specs, "cuda", symmetric_group=dist.group.WORLD if fused_peer else None, world_size=R)
        gen = torch.Generator(device="cuda").manual_seed(7)
        flat.params.copy_((torch.randn(flat.total, device="cuda", generator=gen) * 0.1).bfloat16())
        opt = ZeroAdamW(flat, lr=1e-2, weight_decay=0.1, max_grad_norm=1.0, group=dist.group.WORLD,
                        fused_peer=fused_peer, barrier_timeout_ms=5000.0)
        for step in range(3):
            gr = torch.Generator(device="cuda").manual_seed(100 + step * 10 + r)
            flat.grads.copy_(torch.randn(flat.total, device="cuda", generator=gr))
            torch.cuda.synchronize()
            dist.barrier()
            opt.step()
        _ext.check_status()
        torch.cuda.synchronize()
        dist.barrier()
        results[fused_peer] = (flat.params.clone(), opt.grad_norm.clone())
        assert flat.grads.abs().max().item() == 0.0, "gradients must be cleared by the step"
        opt.close()
    # reference: plain AdamW on the summed gradients, fp32 master
    gen = torch.Generator(device="cuda").manual_seed(7)
    w = (torch.randn(flat.total, device="cuda", generator=gen) * 0.1).bfloat16().float()
    p = torch.nn.Parameter(w.clone())
    dec = torch.zeros_like(w, dtype=torch.bool)
    dec[: flat.decay_end] = True
    m = torch.zeros_like(w)
    vv = torch.zeros_like(w)
    for step in range(3):
        gsum = torch.zeros_like(w)
        for rr in range(R):
            gr = torch.Generator(device="cuda").manual_seed(100 + step * 10 + rr)
            gsum += torch.randn(flat.total, device="cuda", generator=gr)
        norm = gsum.norm()
        gsum = gsum * min(1.0, 1.0 / (norm.item() + 1e-6))
        m = 0.9 * m + 0.1 * gsum
        vv = 0.95 * vv + 0.05 * gsum * gsum
        mh, vh = m / (1 - 0.9 ** (step + 1)), vv / (1 - 0.95 ** (step + 1))
        w = w * (1 - 1e-2 * 0.1 * dec.float()) - 1e-2 * mh / (vh.sqrt() + 1e-8)
    for fp in (True, False):
        got, gn = results[fp]
        assert rel(got, w) < 1e-2, (fp, rel(got, w))
        assert abs(gn.item() - norm.item()) / norm.item() < 1e-3, (fp, gn.item(), norm.item())
    assert torch.equal(results[True][0], results[False][0]) or rel(results[True][0], results[False][0]) < 1e-3
    print(f"rank {r}: zero ok", flush=True)


def case_train(ctx):
    from zenyx_b200.models import LlamaConfig
    from zenyx_b200.ops import _ext
    from zenyx_b200.train import Trainer, TrainerConfig

    R = ctx.world_size
    cfg = LlamaConfig.tiny(n_layers=2, d_model=256, n_heads=4, n_kv_heads=2, ffn_dim=512, vocab_size=512)
    S = 512 * R
    gen = torch.Generator().manual_seed(11)
    tok = torch.randint(0, 512, (R, S), generator=gen)
    curves = {}
    for cp in (R, 1):
        tr = Trainer(cfg, TrainerConfig(lr=2e-3, seq_len=S, global_batch=R, ring_degree=cp, max_grad_norm=1.0, seed=3))
        curves[cp] = [tr.train_step(tok, tok) for _ in range(5)]
        _ext.check_status()
        tr.close()
    if ctx.rank == 0:
        print("loss curves", curves, flush=True)
    a, b = curves[R], curves[1]
    assert a[-1] < a[0] - 0.1, a
    assert all(abs(x - y) < 0.05 for x, y in zip(a, b)), (a, b)   # cp=R and dp=R see the same global batch
    print(f"rank {ctx.rank}: train ok", flush=True)


def case_tp(ctx):
    """all-gather fused into the GEMM (pull warp) and GEMM with a reduce-scatter epilogue (peer red.add),
    against fp32 math on the gathered operands; two calls in a row reuse the buffers."""
    from zenyx_b200.ops import _ext
    from zenyx_b200.parallel.fused_collective import FusedCollectiveContext, allgather_gemm, gemm_reduce_scatter

    R, r = ctx.world_size, ctx.rank
    m, K, N = 384, 512, 768
    fc = FusedCollectiveContext(m, K, N)
    for trial in range(2):
        gen = torch.Generator().manual_seed(100 + trial)
        x_all = torch.randn(R * m, K, generator=gen)
        w = (torch.randn(N, K, generator=gen) / math.sqrt(K))
        y = allgather_gemm(x_all[r * m: (r + 1) * m].cuda().bfloat16(), w.cuda().bfloat16(), fc, fused=True)
        _ext.check_status()
        ref = x_all.bfloat16().float() @ w.bfloat16().float().t()
        assert rel(y.cpu(), ref) < 1e-2, ("allgather_gemm", trial, rel(y.cpu(), ref))
        # row-parallel: each rank holds K/R input features of every row
        Kl = K // R
        xr = x_all[:, r * Kl: (r + 1) * Kl].cuda().bfloat16()
        wr = w[:, r * Kl: (r + 1) * Kl].cuda().bfloat16()
        yr = gemm_reduce_scatter(xr, wr, fc, fused=True)
        _ext.check_status()
        assert rel(yr.cpu(), ref[r * m: (r + 1) * m]) < 1e-2, ("gemm_reduce_scatter", trial, rel(yr.cpu(), ref[r * m: (r + 1) * m]))
        # the automatic choice (fused or library collective, by size and rank count) gives the same numbers
        ya = allgather_gemm(x_all[r * m: (r + 1) * m].cuda().bfloat16(), w.cuda().bfloat16(), fc)
        yra = gemm_reduce_scatter(xr, wr, fc)
        assert rel(ya.cpu(), ref) < 1e-2 and rel(yra.cpu(), ref[r * m: (r + 1) * m]) < 1e-2
    fc.close()
    print(f"rank {r}: tp ok", flush=True)


def main():
    from zenyx_b200.parallel.communication import init_distributed_from_env

    ctx = init_distributed_from_env(timeout_seconds=120)
    cases = sys.argv[1:] or ["ring", "zero", "train"]
    for c in cases:
        globals()["case_" + c](ctx)
        torch.cuda.synchronize()
        dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
