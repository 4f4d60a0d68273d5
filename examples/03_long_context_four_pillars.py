"""Example 03: the long-context configuration and its four pillars.

    python examples/03_long_context_four_pillars.py                       # one process: plans + a small run
    python -m torch.distributed.run --nproc-per-node 8 examples/03_long_context_four_pillars.py --train

The counterpart of the reference's expert example (examples/03_expert_tpu_v5e8_training.py), which
configures a 1M-token run on eight accelerators: Belady KV tiering, FP8 KV quantisation, the dynamic
ring-degree curriculum and sparse ring attention. Here every pillar is a working component: the
example prints what the planner and each pillar decide for the 8B / 8-GPU configuration, runs the
attention modules on the device that is present, and with ``--train`` under torchrun trains a small
model with the ring curriculum over the GPUs it was given.
"""
import argparse
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
from zenyx_b200.models import LlamaConfig  # noqa: E402
from zenyx_b200.planner import plan  # noqa: E402
from zenyx_b200.train import Trainer, TrainerConfig  # noqa: E402
from zenyx_b200.train.belayd_kv_cache_tiering import BeladyKVCacheTieringManager  # noqa: E402
from zenyx_b200.train.dynamic_ring_curriculum import RingDegreeScheduler  # noqa: E402
from zenyx_b200.train.fp8_kv_quantization import FP8KVQuantizer, QuantizedRingAttention  # noqa: E402
from zenyx_b200.train.sparse_ring_attention import SparsePattern, SparseRingAttention  # noqa: E402


def describe():
    cfg = LlamaConfig.llama3_8b()
    print("[plan] 8B shape, 32K context, 8 sequences per step:")
    for n in (1, 2, 4, 8):
        print(f"   {n} GPU(s): {plan(cfg, 32768, 8, n, hbm_bytes=192e9, memory_fraction=0.93).describe()}")
    print(f"   262,144 tokens on 8 GPUs (ring forced by memory): "
          f"{plan(cfg, 262144, 8, 8, hbm_bytes=192e9, memory_fraction=0.93).describe()}")
    mgr = BeladyKVCacheTieringManager(num_devices=8, context_length=1 << 20, num_layers=8, hbm_budget_bytes=1 << 30,
                                      simulate=True)
    p = mgr.plan()
    print(f"[pillar 1] KV tiering, 1M tokens, 8 layers, 1 GB of HBM for {mgr.total_kv_bytes() / 2**30:.1f} GB of KV per GPU: "
          f"{p.misses} misses in {len(p.ids)} accesses (LRU: {mgr.lru_baseline()['misses']})")
    q = FP8KVQuantizer(num_kv_heads=8, head_dim=128)
    x = torch.randn(1, 1024, 8, 128).bfloat16()
    print(f"[pillar 2] e4m3 KV with per-head, per-128-token scales: {q.compression_ratio:.2f}x smaller, "
          f"relative error {q.relative_error(x):.4f}")
    sched = RingDegreeScheduler(world_size=8)
    print(f"[pillar 3] ring degree over the first 400 steps: {[sched.degree_at(s) for s in range(0, 400, 50)]}")
    pat = SparsePattern(window_tokens=4096, global_every=64)
    print(f"[pillar 4] 4096-token window + every 64th block global at 262,144 tokens keeps "
          f"{100 * pat.density(262144):.2f} % of the score tiles")


def small_run():
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    torch.manual_seed(0)
    B, S, Hq, Hkv, D = 1, 1024, 4, 2, 128
    qkv = [torch.randn(B, S, h, D, device=dev).bfloat16() for h in (Hq, Hkv, Hkv)]
    sparse = SparseRingAttention(SparsePattern(window_tokens=256, global_every=4), Hq, Hkv, D)
    quant = QuantizedRingAttention(Hq, Hkv, D)
    o_s, o_q = sparse(*qkv), quant(*qkv)
    print(f"[run] sparse ring attention output {tuple(o_s.shape)}, FP8-KV ring attention output {tuple(o_q.shape)} on {dev}")


def train(steps: int):
    import torch.distributed as dist

    from zenyx_b200.parallel.communication import init_distributed_from_env

    ctx = init_distributed_from_env()
    world = ctx.world_size
    cfg = LlamaConfig.tiny(n_layers=2, d_model=256, n_heads=4, n_kv_heads=2, ffn_dim=512, vocab_size=512)
    seq = 256 * 2 * world
    degrees = [d for d in (1, 2, 4, 8) if d <= world]
    cur = RingDegreeScheduler(world_size=world) if world > 1 else None
    tr = Trainer(cfg, TrainerConfig(lr=2e-3, seq_len=seq, global_batch=world, ring_degree=world, ring_degrees=degrees,
                                    curriculum=cur, max_grad_norm=1.0))
    gen = torch.Generator().manual_seed(0)
    for step in range(steps):
        tok = torch.randint(0, 512, (world, seq), generator=gen)
        loss = tr.train_step(tok, torch.roll(tok, -1, dims=1))
        if ctx.rank == 0:
            print(f"step {step}: loss {loss:.4f}, ring degree {tr.engine.ring_degree}")
    tr.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--train", action="store_true")
    ap.add_argument("--steps", type=int, default=6)
    a = ap.parse_args()
    if a.train:
        train(a.steps)
    else:
        describe()
        small_run()
