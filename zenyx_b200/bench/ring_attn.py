"""Standalone causal ring attention benchmark (forward + backward), the second headline metric.

    python -m zenyx_b200.bench.ring_attn                       (1 GPU, ring degree 1)
    python -m torch.distributed.run --nproc-per-node R -m zenyx_b200.bench.ring_attn

B=1, 32 query heads, 8 KV heads, head_dim 128, total sequence 131072 split over the ring with
load-balanced zigzag chunking; Q/K/V and dO ~ N(0,1). Reports device-timed ms (max over ranks) and
TFLOP/s on the algorithmic count 4*S^2*d*Hq/2 (forward) and 2.5x that (backward), whole job and per
GPU, plus the fraction of the roofline max(FLOPs / measured GEMM peak, NVLink bytes / 770 GB/s).
``--check`` additionally verifies a 16K slice against an fp32 reference on one GPU.
"""
from __future__ import annotations

import argparse
import json
import math

import torch
import torch.distributed as dist


def slice_check(ring, q, k, v, do, o, lse, dq, dk, dv, scale, mask, n_check=16384):
    """fp32 reference on two slices of the global sequence, computed on every rank from all-reduced copies:

    * the FIRST ``n_check`` positions: O, LSE and dQ of those queries only involve keys of the same slice;
    * the LAST ``n_check`` positions: dK and dV of those keys only receive from queries of the same slice
      (their softmax runs over the whole sequence, so the reference takes the kernels' LSE and
      delta = rowsum(dO * O) for those rows, which the first slice has verified in kind).

    Returns relative Frobenius errors and maximum absolute errors per tensor."""
    R, S = ring.degree, ring.seq_len
    dev = q.device
    Lc = q.shape[1] // len(ring.positions())

    def collect(x, lo, hi, token_dim=1):
        """[.., hi - lo tokens, ..] in global order: each rank places the tokens it owns, the rest are zeros."""
        shape = list(x.shape)
        shape[token_dim] = hi - lo
        out = torch.zeros(shape, device=dev, dtype=torch.float32)
        for ci, p0 in enumerate(ring.positions()):
            a, b = max(p0, lo), min(p0 + Lc, hi)
            if a < b:
                src = x.narrow(token_dim, ci * Lc + (a - p0), b - a).float()
                out.narrow(token_dim, a - lo, b - a).copy_(src)
        if R > 1:
            dist.all_reduce(out)
        return out

    def masked_scores(qs, ks, q0, k0):
        qpos = torch.arange(q0, q0 + qs.shape[1], device=dev)
        kpos = torch.arange(k0, k0 + ks.shape[1], device=dev)
        keep = kpos[None, :] <= qpos[:, None]
        if mask.window_blocks > 0:
            qb, kb = qpos[:, None] // 128, kpos[None, :] // 128
            win = (qb - kb).abs() < mask.window_blocks
            glob = (kb % mask.global_every == 0) if mask.global_every > 0 else torch.zeros_like(win)
            keep = keep & (win | glob)
        return keep

    def err(a, b):
        return {"rel": round(float((a - b).norm() / (b.norm() + 1e-20)), 5), "max_abs": round(float((a - b).abs().max()), 5)}

    G = q.shape[2] // k.shape[2]
    res = {"slice_tokens": n_check}
    # ---- first slice: O, LSE, dQ
    qf, dof = collect(q, 0, n_check), collect(do, 0, n_check)
    kf, vf = collect(k, 0, n_check), collect(v, 0, n_check)
    of, dqf = collect(o, 0, n_check), collect(dq, 0, n_check)
    lsef = collect(lse, 0, n_check, token_dim=2)
    keep = masked_scores(qf, kf, 0, 0)
    o_ref, dq_ref, lse_ref = torch.empty_like(of), torch.empty_like(dqf), torch.empty_like(lsef)
    for h in range(q.shape[2]):
        s = (qf[0, :, h] @ kf[0, :, h // G].T) * scale
        s = s.masked_fill(~keep, float("-inf"))
        lse_h = torch.logsumexp(s, dim=-1)
        p = torch.exp(s - lse_h[:, None])
        oh = p @ vf[0, :, h // G]
        dp = dof[0, :, h] @ vf[0, :, h // G].T
        ds = p * (dp - (dof[0, :, h] * oh).sum(-1, keepdim=True))
        o_ref[0, :, h], lse_ref[0, h], dq_ref[0, :, h] = oh, lse_h, (ds @ kf[0, :, h // G]) * scale
    res["o"], res["lse"], res["dq"] = err(of, o_ref), err(lsef, lse_ref), err(dqf, dq_ref)
    # ---- last slice: dK, dV
    lo = S - n_check
    ql, dol, ol = collect(q, lo, S), collect(do, lo, S), collect(o, lo, S)
    kl, vl = collect(k, lo, S), collect(v, lo, S)
    dkl, dvl = collect(dk, lo, S), collect(dv, lo, S)
    lsel = collect(lse, lo, S, token_dim=2)
    keep = masked_scores(ql, kl, lo, lo)
    dk_ref, dv_ref = torch.zeros_like(dkl), torch.zeros_like(dvl)
    for h in range(q.shape[2]):
        s = (ql[0, :, h] @ kl[0, :, h // G].T) * scale
        p = torch.exp(s - lsel[0, h][:, None]).masked_fill(~keep, 0.0)
        dp = dol[0, :, h] @ vl[0, :, h // G].T
        ds = p * (dp - (dol[0, :, h] * ol[0, :, h]).sum(-1, keepdim=True))
        dv_ref[0, :, h // G] += p.T @ dol[0, :, h]
        dk_ref[0, :, h // G] += (ds.T @ ql[0, :, h]) * scale
    res["dk"], res["dv"] = err(dkl, dk_ref), err(dvl, dv_ref)
    res["ok"] = all(res[n]["rel"] < 2e-2 for n in ("o", "dq", "dk", "dv")) and res["lse"]["max_abs"] < 2e-2
    return res


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--seq-len", type=int, default=131072)
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--check", action="store_true")
    ap.add_argument("--window-tokens", type=int, default=0, help="> 0: block-sparse (window + --global-every)")
    ap.add_argument("--global-every", type=int, default=64)
    ap.add_argument("--fp8-kv", action="store_true",
                    help="K/V in the e4m3 cache format (per head and 128-token block scales): codes in the peer slots and on NVLink")
    args = ap.parse_args(argv)

    from zenyx_b200.bench.kernels import peaks
    from zenyx_b200.ops import _ext
    from zenyx_b200.ops.attention import (MaskSpec, RingContext, ring_attn_backward, ring_attn_forward, shard_sequence)
    from zenyx_b200.parallel.communication import init_distributed_from_env

    ctx = init_distributed_from_env()
    R, r, dev = ctx.world_size, ctx.rank, ctx.device
    B, S, Hq, Hkv, D = 1, args.seq_len, 32, 8, 128
    Sl = S // R
    scale = 1 / math.sqrt(D)
    mask = MaskSpec(True, args.window_tokens // 128, args.global_every if args.window_tokens else 0)
    g = torch.Generator(device=dev).manual_seed(100 + r)
    q = torch.randn(B, Sl, Hq, D, device=dev, generator=g).bfloat16()
    do = torch.randn(B, Sl, Hq, D, device=dev, generator=g).bfloat16()
    peer = None
    if R > 1:
        from zenyx_b200.parallel.peer import RingBuffers

        peer = RingBuffers((B, Sl, Hkv, D), group=None, fp8_block_tokens=128 if args.fp8_kv else 0)
        if args.fp8_kv:
            k = torch.randn(B, Sl, Hkv, D, device=dev, generator=g).bfloat16()
            v = torch.randn(B, Sl, Hkv, D, device=dev, generator=g).bfloat16()
        else:
            k, v = peer.kv_views(r, 0)
            k.copy_(torch.randn(B, Sl, Hkv, D, device=dev, generator=g).bfloat16())
            v.copy_(torch.randn(B, Sl, Hkv, D, device=dev, generator=g).bfloat16())
    else:
        k = torch.randn(B, Sl, Hkv, D, device=dev, generator=g).bfloat16()
        v = torch.randn(B, Sl, Hkv, D, device=dev, generator=g).bfloat16()
        if args.fp8_kv:   # one GPU: no slots, the cache format is a round trip
            from zenyx_b200.train.fp8_kv_quantization import FP8KVQuantizer

            qz = FP8KVQuantizer(Hkv, D, 128)
            k, v = qz.roundtrip(k), qz.roundtrip(v)
    ring = RingContext(rank=r, degree=R, seq_len=S, peer=peer, mask=mask)

    def sync():
        if R > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn):
        for _ in range(args.warmup):
            fn()
        ts = []
        for _ in range(args.iters):
            sync()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            out = fn()
            e1.record()
            sync()
            t = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
            if R > 1:
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ts.append(float(t.item()))
        ts.sort()
        return ts[len(ts) // 2], out

    ms_f, (o, lse) = timed(lambda: ring_attn_forward(ring, q, k, v, scale, 0))
    ms_b, _ = timed(lambda: ring_attn_backward(ring, q, k, v, o, do, lse, scale, 0))
    _ext.check_status()
    density = 1.0
    if args.window_tokens:
        from zenyx_b200.train.sparse_ring_attention import SparsePattern

        density = SparsePattern(window_tokens=args.window_tokens, global_every=args.global_every).density(S)
    f_fwd = 4.0 * S * S * D * Hq * 0.5 * density
    f_bwd = 2.5 * f_fwd
    pk = peaks()
    kv_bytes = 2 * Sl * Hkv * D * (1 if args.fp8_kv else 2)                   # K and V of one rank as they travel
    nvlink_s = (2 * kv_bytes + 2 * Sl * Hkv * D * 4) * (R - 1) / 770e9        # fwd pull + bwd pull + fp32 dK/dV push
    roof_s = max((f_fwd + f_bwd) / R / (pk["tflops_sustained"] * 1e12), nvlink_s)
    rec = {"metric": "ring-attn fwd+bwd TFLOP/s", "ring_degree": R, "seq_len": S, "heads": [Hq, Hkv], "head_dim": D,
           "layout": "zigzag", "kv_format": "e4m3 + fp32 scale per (head, 128 tokens)" if args.fp8_kv else "bf16",
           "mask": "causal" + (f"+window{args.window_tokens}+global{args.global_every}" if args.window_tokens else ""),
           "fwd_ms": round(ms_f, 3), "bwd_ms": round(ms_b, 3),
           "fwd_tflops": round(f_fwd / ms_f / 1e9, 1), "bwd_tflops": round(f_bwd / ms_b / 1e9, 1),
           "value": round((f_fwd + f_bwd) / (ms_f + ms_b) / 1e9, 1), "unit": "TFLOP/s (whole job)",
           "per_gpu_tflops": round((f_fwd + f_bwd) / (ms_f + ms_b) / 1e9 / R, 1),
           "roofline_ms": round(roof_s * 1e3, 2), "frac_of_roofline": round(roof_s * 1e3 / (ms_f + ms_b), 3),
           "peaks": pk["source"], "timing": "CUDA events, max over ranks, median of %d" % args.iters}
    if args.check:
        dq, dk, dv = ring_attn_backward(ring, q, k, v, o, do, lse, scale, 0)
        k_ref, v_ref = k, v
        if args.fp8_kv:   # the reference attends what the cache format holds
            from zenyx_b200.train.fp8_kv_quantization import FP8KVQuantizer

            qz = FP8KVQuantizer(Hkv, D, 128)
            k_ref, v_ref = qz.roundtrip(k), qz.roundtrip(v)
        chk = slice_check(ring, q, k_ref, v_ref, do, o, lse, dq, dk, dv, scale, mask, n_check=min(16384, S // 2))
        _ext.check_status()
        if r == 0:
            rec["check"] = chk
    if r == 0:
        print(json.dumps(rec), flush=True)
    if peer is not None:
        peer.close()
    if R > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
