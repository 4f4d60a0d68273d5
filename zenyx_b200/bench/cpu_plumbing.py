"""CPU plumbing benchmark: the README ``SimpleTransformer`` through the public ``Trainer`` on CPU, fp32.

    python -m zenyx_b200.bench.cpu_plumbing                     # this framework
    python -m zenyx_b200.bench.cpu_plumbing --impl reference    # the unmodified reference's Trainer

vocab 10000, d_model 768, 12 post-LN encoder layers (12 heads, FFN 2048, ReLU, dropout 0.1), batch 8,
sequence 512, tokens and targets uniform from seed 0, cross-entropy, AdamW lr 1e-4, 20 steps, with a
``BeladyKVCacheTieringManager(num_devices=8, context_length=4096, num_layers=12)`` planned in
simulation mode beside it (this framework's arm only: the installed reference package has no such
module). Prints one JSON line: tokens/s over steps 2..N, first and final loss.
The reference's counterpart is its README quick start (README.md:60-110) run through
zenyx/train/trainer.py:16-57.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

import torch
import torch.nn as nn


class _TokenCE(nn.Module):
    def forward(self, logits, target):
        return nn.functional.cross_entropy(logits.reshape(-1, logits.shape[-1]), target.reshape(-1))


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--impl", default="zenyx_b200", choices=["zenyx_b200", "reference"])
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--seq-len", type=int, default=512)
    args = ap.parse_args(argv)
    torch.manual_seed(0)
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    extra = {}
    if args.impl == "reference":
        ref = os.path.join(root, "baseline", "_ref")
        if not os.path.isdir(os.path.join(ref, "zenyx")):
            print(json.dumps({"impl": "reference", "unavailable": "reference package is not installed under baseline/_ref"}))
            return
        sys.path.insert(0, ref)
        from zenyx.train import Trainer, TrainerConfig  # the reference

        sys.path.insert(0, root)
        from zenyx_b200.models.simple_transformer import SimpleTransformer  # plain nn.Module, stock PyTorch layers
    else:
        from zenyx_b200.models.simple_transformer import SimpleTransformer
        from zenyx_b200.train import Trainer, TrainerConfig
        from zenyx_b200.train.belayd_kv_cache_tiering import BeladyKVCacheTieringManager

        mgr = BeladyKVCacheTieringManager(num_devices=8, context_length=4096, num_layers=12, simulate=True)
        plan = mgr.plan()
        extra["kv_tiering_plan"] = {"accesses": len(plan.ids), "hits": plan.hits, "misses": plan.misses,
                                    "lru_misses": mgr.lru_baseline()["misses"]}
    model = SimpleTransformer()
    trainer = Trainer(model, TrainerConfig(lr=1e-4))
    crit = _TokenCE()
    gen = torch.Generator().manual_seed(0)
    x = torch.randint(0, 10000, (args.batch, args.seq_len), generator=gen)
    y = torch.randint(0, 10000, (args.batch, args.seq_len), generator=gen)
    losses, t_first = [], None
    for step in range(args.steps):
        if step == 1:
            t_first = time.perf_counter()
        losses.append(float(trainer.train_step(x, y, crit)))
    dt = time.perf_counter() - t_first
    tokens = args.batch * args.seq_len * (args.steps - 1)
    print(json.dumps({"metric": "CPU plumbing tokens/s (README SimpleTransformer, fp32)", "impl": args.impl,
                      "value": round(tokens / dt, 1), "unit": "tokens/s", "steps": args.steps,
                      "s_per_step": round(dt / (args.steps - 1), 3), "first_loss": round(losses[0], 4),
                      "final_loss": round(losses[-1], 4), "threads": torch.get_num_threads(), **extra}), flush=True)


if __name__ == "__main__":
    main()
