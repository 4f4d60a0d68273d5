"""Accuracy of attention over FP8 (e4m3) K/V against bf16 K/V and against fp32 math.

    python -m zenyx_b200.bench.fp8_kv_error [--seq-len 4096] [--window-tokens 1024 --global-every 4]

K and V are quantised per KV head and per 128-token block with a dynamic absmax scale
(``FP8KVQuantizer``), the attention itself runs the same kernels (bf16 tensor cores; fp32 fall-backs
on CPU). Three outputs are compared on the same random Q/K/V: fp32 reference, bf16 K/V, FP8 K/V; one
JSON line with relative errors (Frobenius) and the worst absolute difference. The reference claims
"<0.1 % accuracy impact" for this scheme without code or measurement (README.md:156-160).
"""
from __future__ import annotations

import argparse
import json
import math

import torch


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--seq-len", type=int, default=4096)
    ap.add_argument("--heads", type=int, default=8)
    ap.add_argument("--kv-heads", type=int, default=2)
    ap.add_argument("--window-tokens", type=int, default=0)
    ap.add_argument("--global-every", type=int, default=0)
    ap.add_argument("--scale-inputs", type=float, default=1.0, help="standard deviation of Q, K, V")
    args = ap.parse_args(argv)
    from zenyx_b200.ops.attention import MaskSpec, flash_attention
    from zenyx_b200.train.fp8_kv_quantization import FP8KVQuantizer

    dev = "cuda" if torch.cuda.is_available() else "cpu"
    torch.manual_seed(0)
    B, S, Hq, Hkv, D = 1, args.seq_len, args.heads, args.kv_heads, 128
    q = (torch.randn(B, S, Hq, D, device=dev) * args.scale_inputs).bfloat16()
    k = (torch.randn(B, S, Hkv, D, device=dev) * args.scale_inputs).bfloat16()
    v = (torch.randn(B, S, Hkv, D, device=dev) * args.scale_inputs).bfloat16()
    sparse = None
    if args.window_tokens:
        sparse = MaskSpec(True, args.window_tokens // 128, args.global_every)
    qz = FP8KVQuantizer(Hkv, D)
    k8, v8 = qz.roundtrip(k), qz.roundtrip(v)
    o_bf16 = flash_attention(q, k, v, causal=True, sparse=sparse).float()
    o_fp8 = flash_attention(q, k8, v8, causal=True, sparse=sparse).float()
    # fp32 reference with the same mask, in blocks of queries to bound memory
    g = Hq // Hkv
    qf = q.float().permute(0, 2, 1, 3)
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(g, 1)
    vf = v.float().permute(0, 2, 1, 3).repeat_interleave(g, 1)
    pos = torch.arange(S, device=dev)
    o_ref = torch.empty_like(qf)
    for s0 in range(0, S, 1024):
        s1 = min(S, s0 + 1024)
        sc = torch.einsum("bhqd,bhkd->bhqk", qf[:, :, s0:s1], kf) / math.sqrt(D)
        mask = pos[None, :] <= pos[s0:s1, None]
        if sparse is not None:
            qb, kb = (pos[s0:s1] // 128)[:, None], (pos // 128)[None, :]
            keep = (qb - kb).abs() < sparse.window_blocks
            if sparse.global_every > 0:
                keep |= (kb % sparse.global_every) == 0
            mask &= keep
        sc = sc.masked_fill(~mask, float("-inf"))
        o_ref[:, :, s0:s1] = torch.einsum("bhqk,bhkd->bhqd", torch.softmax(sc, -1), vf)
    o_ref = o_ref.permute(0, 2, 1, 3)

    def rel(a, b):
        return float((a - b).norm() / b.norm())

    print(json.dumps({
        "metric": "attention output error with e4m3 K/V", "device": dev, "seq_len": S, "heads": [Hq, Hkv], "head_dim": D,
        "mask": "causal" + (f"+window{args.window_tokens}+global{args.global_every}" if sparse else ""),
        "input_std": args.scale_inputs,
        "kv_roundtrip_rel_error": {"k": round(qz.relative_error(k), 5), "v": round(qz.relative_error(v), 5)},
        "bf16_kv_vs_fp32": round(rel(o_bf16, o_ref), 5), "fp8_kv_vs_fp32": round(rel(o_fp8, o_ref), 5),
        "fp8_kv_vs_bf16_kv": round(rel(o_fp8, o_bf16), 5),
        "max_abs_diff_fp8_vs_bf16": round(float((o_fp8 - o_bf16).abs().max()), 5),
        "kv_bytes_ratio": round(qz.compression_ratio, 3),
    }), flush=True)


if __name__ == "__main__":
    main()
