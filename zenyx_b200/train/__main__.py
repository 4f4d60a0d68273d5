"""``python -m zenyx_b200.train``: command-line training on synthetic tokens.

The reference promises CLI tools as future work (README.md:494) and quotes the flags of a deleted
script, ``--model-size --batch-size --num-epochs`` (README.md:229-234); those three are accepted here.
Launch with ``python -m torch.distributed.run --nproc-per-node N -m zenyx_b200.train ...`` for N GPUs.
"""
from __future__ import annotations

import argparse
import json

import torch

from ..models import LlamaConfig
from .dynamic_ring_curriculum import RingDegreeScheduler
from .loop import LoopConfig, run
from .lr_schedule import warmup_cosine
from .trainer import Trainer, TrainerConfig

SIZES = {
    "tiny": dict(n_layers=2, d_model=256, n_heads=2, n_kv_heads=1, ffn_dim=512, vocab_size=4096),
    "small": dict(n_layers=8, d_model=1024, n_heads=8, n_kv_heads=2, ffn_dim=2816, vocab_size=32768),
    "medium": dict(n_layers=16, d_model=2048, n_heads=16, n_kv_heads=4, ffn_dim=5632, vocab_size=65536),
    "large": dict(n_layers=32, d_model=4096, n_heads=32, n_kv_heads=8, ffn_dim=14336, vocab_size=128256),
}


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(prog="python -m zenyx_b200.train")
    ap.add_argument("--model-size", default="tiny", choices=sorted(SIZES))
    ap.add_argument("--batch-size", type=int, default=8, help="sequences per optimizer step (global)")
    ap.add_argument("--num-epochs", type=int, default=1)
    ap.add_argument("--steps-per-epoch", type=int, default=10)
    ap.add_argument("--seq-len", type=int, default=1024)
    ap.add_argument("--lr", type=float, default=3e-4)
    ap.add_argument("--ring-degree", type=int, default=1)
    ap.add_argument("--curriculum", action="store_true", help="ramp the ring degree 2 -> ... -> --ring-degree")
    ap.add_argument("--checkpoint-dir", default=None)
    ap.add_argument("--metrics", default=None)
    args = ap.parse_args(argv)

    mc = LlamaConfig.tiny(**SIZES[args.model_size])
    steps = args.num_epochs * args.steps_per_epoch
    import os

    world = int(os.environ.get("WORLD_SIZE", "1"))
    cur = None
    if args.curriculum and args.ring_degree > 1:
        cur = RingDegreeScheduler(min_degree=min(2, args.ring_degree), max_degree=args.ring_degree,
                                  ramp_steps=max(1, steps // 2), world_size=world)
    tcfg = TrainerConfig(lr=args.lr, seq_len=args.seq_len, global_batch=args.batch_size, ring_degree=args.ring_degree,
                         curriculum=cur, max_grad_norm=1.0, weight_decay=0.1,
                         lr_schedule=warmup_cosine(args.lr, max(1, steps // 10), steps, args.lr * 0.1))
    trainer = Trainer(mc, tcfg)
    gen = torch.Generator().manual_seed(0)

    def data():
        while True:
            tok = torch.randint(0, mc.vocab_size, (args.batch_size, args.seq_len + 1), generator=gen)
            yield tok[:, :-1].contiguous(), tok[:, 1:].contiguous()

    recs = run(trainer, data(), None, LoopConfig(steps=steps, log_every=1, checkpoint_dir=args.checkpoint_dir,
                                                 metrics_path=args.metrics,
                                                 tokens_per_step=args.batch_size * args.seq_len))
    if trainer.ctx.rank == 0 and recs:
        print(json.dumps({"first_loss": recs[0]["loss"], "last_loss": recs[-1]["loss"], "steps": len(recs)}))
    trainer.close()


if __name__ == "__main__":
    main()
