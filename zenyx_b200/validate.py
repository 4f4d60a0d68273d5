"""``python -m zenyx_b200.validate``: a quick check of the four long-context pillars and the core
components on whatever device is present (the reference's README points at
``test/validate_zenyx_four_pillars.py``, README.md:46-48,199, which is not in its tree).

Each check prints one line and the process exits non-zero if any fails. On a machine without a GPU the
kernels' CPU fallbacks run; with a GPU the CUDA kernels are used and must be loadable.
"""
from __future__ import annotations

import sys
import traceback

import torch


def _belady():
    from zenyx_b200.train.belayd_kv_cache_tiering import BeladyKVCacheTieringManager

    m = BeladyKVCacheTieringManager(num_devices=8, context_length=1 << 16, num_layers=4, hbm_budget_bytes=64 << 20,
                                    tier_block_tokens=1024, simulate=True)
    p, lru = m.plan(), m.lru_baseline()
    assert p.misses <= lru["misses"], (p.misses, lru)
    return f"{len(p.ids)} accesses, Belady misses {p.misses} <= LRU misses {lru['misses']}"


def _fp8():
    from zenyx_b200.train.fp8_kv_quantization import FP8KVQuantizer

    q = FP8KVQuantizer(num_kv_heads=2, head_dim=128)
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    x = torch.randn(1, 256, 2, 128, device=dev).bfloat16()
    err = q.relative_error(x)
    ratio = q.compression_ratio
    assert err < 0.05 and abs(ratio - 2.0) < 0.1, (err, ratio)
    return f"relative error {err:.4f}, compression {ratio:.2f}x"


def _curriculum():
    from zenyx_b200.train.dynamic_ring_curriculum import RingDegreeScheduler

    s = RingDegreeScheduler(world_size=8)
    degs = [s.degree_at(t) for t in range(0, 400, 50)]
    assert degs[0] <= degs[-1] and set(degs) <= {1, 2, 4, 8}, degs
    return f"ring degree over steps 0..350: {degs}"


def _sparse():
    from zenyx_b200.train.sparse_ring_attention import SparsePattern

    p = SparsePattern(window_tokens=4096, global_every=64)
    d = p.density(1 << 18)
    assert 0.0 < d < 0.2, d
    return f"kept tiles at 256K tokens: {100 * d:.2f} % of the causal triangle's square"


def _attention():
    from zenyx_b200.ops.attention import flash_attention

    dev = "cuda" if torch.cuda.is_available() else "cpu"
    q = torch.randn(1, 256, 4, 128, device=dev).bfloat16()
    k = torch.randn(1, 256, 2, 128, device=dev).bfloat16()
    v = torch.randn(1, 256, 2, 128, device=dev).bfloat16()
    o = flash_attention(q, k, v, causal=True)
    ref = torch.nn.functional.scaled_dot_product_attention(q.float().transpose(1, 2), k.float().transpose(1, 2).repeat_interleave(2, 1),
                                                           v.float().transpose(1, 2).repeat_interleave(2, 1), is_causal=True)
    err = (o.float().transpose(1, 2) - ref).abs().max().item()
    assert err < 3e-2, err
    return f"flash attention on {dev}: max abs error {err:.4f} vs fp32"


def _trainer():
    from zenyx_b200.models import LlamaConfig
    from zenyx_b200.train import Trainer, TrainerConfig

    cfg = LlamaConfig.tiny(n_layers=2, d_model=256, n_heads=2, n_kv_heads=1, ffn_dim=512, vocab_size=512)
    tr = Trainer(cfg, TrainerConfig(lr=2e-3, seq_len=256, global_batch=2))
    tok = torch.randint(0, 512, (2, 256))
    losses = [tr.train_step(tok, tok) for _ in range(4)]
    tr.close()
    assert losses[-1] < losses[0], losses
    return f"loss {losses[0]:.3f} -> {losses[-1]:.3f} in 4 steps"


CHECKS = [("Belady KV tiering plan", _belady), ("FP8 KV quantiser", _fp8), ("ring-degree curriculum", _curriculum),
          ("sparse ring pattern", _sparse), ("flash attention", _attention), ("Trainer on a tiny Llama", _trainer)]


def main() -> int:
    failed = 0
    for name, fn in CHECKS:
        try:
            print(f"[ ok ] {name}: {fn()}", flush=True)
        except Exception as e:  # noqa: BLE001
            failed += 1
            print(f"[FAIL] {name}: {type(e).__name__}: {e}", flush=True)
            traceback.print_exc()
    print(f"{len(CHECKS) - failed} of {len(CHECKS)} checks passed")
    return 1 if failed else 0


if __name__ == "__main__":
    sys.exit(main())
