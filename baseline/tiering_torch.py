"""Same-box baseline of the KV tiering stress (``zenyx_b200.bench.kv_tiering``): the UNMODIFIED reference
``zenyx.streaming.KVTierManager`` (zenyx/streaming/kv_tiering.py:18-66: an LRU ``OrderedDict`` per tier, pageable
``tensor.cpu()`` / ``.to(device)`` copies on the current stream, no schedule, no prefetch) serving the same access
trace, with stock ``scaled_dot_product_attention`` as the consumer of every block.

    python -m baseline.tiering_torch [--context 1048576 --ring 8 --layers 8 --block-tokens 4096 --hbm-gb 16]

The trace (which block of this rank's K/V share is touched when) comes from this package's
``RingAttentionAccessSequence``; the reference has no generator for it (its ``build_ring_timeline`` lists
``range(num_blocks)``), so both arms replay identical accesses. ``t0_capacity`` is the HBM budget in blocks,
``t1_capacity`` the host-DRAM budget. Prints one JSON line with the fields of the benchmark it is the baseline for.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--context", type=int, default=1 << 20)
    ap.add_argument("--ring", type=int, default=8)
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--block-tokens", type=int, default=4096)
    ap.add_argument("--hbm-gb", type=float, default=16.0)
    ap.add_argument("--q-tokens", type=int, default=8192)
    ap.add_argument("--steps", type=int, default=2)
    args = ap.parse_args(argv)
    sys.path.insert(0, os.path.join(HERE, "_ref"))
    try:
        import torch
        import torch.nn.functional as F
        from zenyx.streaming import KVTierManager     # the reference
    except Exception as e:  # noqa: BLE001
        print(json.dumps({"impl": "reference KVTierManager", "unavailable": f"{type(e).__name__}: {e}"[:200]}), flush=True)
        return
    from zenyx_b200.train.belayd_kv_cache_tiering import RingAttentionAccessSequence

    dev = torch.device("cuda")
    Hq, Hkv, D, bt = 32, 8, 128, args.block_tokens
    local_tokens = args.context // args.ring
    blocks_per_layer = local_tokens // bt
    block_bytes = 2 * bt * Hkv * D * 2
    t0_cap = max(1, int(args.hbm_gb * (1 << 30)) // block_bytes)
    ids = RingAttentionAccessSequence(args.ring, args.layers, blocks_per_layer, zigzag=True,
                                      seq_len=args.context).block_ids(0)
    mgr = KVTierManager(t0_capacity=t0_cap, t1_capacity=args.layers * blocks_per_layer)
    gen = torch.Generator(device=dev).manual_seed(0)
    for bid in range(args.layers * blocks_per_layer):
        mgr.put(bid, torch.randn(2, bt, Hkv, D, device=dev, generator=gen).bfloat16())
    q = torch.randn(1, Hq, args.q_tokens, D, device=dev, generator=gen).bfloat16()
    times, loaded = [], 0
    for _ in range(args.steps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for bid in ids:
            hit = bid in mgr.t0
            blk = mgr.prefetch_to_t0(bid, dev)
            loaded += 0 if hit else block_bytes
            k, v = blk[0].unsqueeze(0).transpose(1, 2), blk[1].unsqueeze(0).transpose(1, 2)
            F.scaled_dot_product_attention(q, k, v, enable_gqa=True)
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    ms = min(times)
    flops = 4.0 * args.q_tokens * bt * D * Hq * len(ids)
    print(json.dumps({"metric": "KV tiering stress step time", "impl": "reference KVTierManager (LRU, synchronous copies) + SDPA",
                      "value": round(ms, 2), "unit": "ms", "higher_is_better": False, "step_ms_all": [round(t, 2) for t in times],
                      "context_tokens": args.context, "ring": args.ring, "layers": args.layers, "block_tokens": bt,
                      "hbm_budget_blocks": t0_cap, "accesses_per_step": len(ids), "bytes_h2d_total": loaded,
                      "attention_tflops": round(flops / ms / 1e9, 1)}), flush=True)


if __name__ == "__main__":
    main()
