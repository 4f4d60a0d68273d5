"""Example 02: fine-tuning the Llama-shaped model with a schedule, checkpoints and resume.

    python examples/02_finetune_with_checkpoints.py [--steps 12] [--dir /tmp/zx_example02]

Mirrors the reference's intermediate example (examples/02_intermediate_finetuning.py): a "pre-trained"
model is saved, loaded back chunk by chunk, trained further with warm-up + cosine decay and gradient
clipping, checkpointed on the way, and a second run resumes from the last checkpoint. On a GPU the
model runs on the sm_100a kernels; on CPU on their fp32 fallbacks.
"""
import argparse
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
from zenyx_b200 import loader  # noqa: E402
from zenyx_b200.models import LlamaConfig  # noqa: E402
from zenyx_b200.train import Trainer, TrainerConfig, loop, lr_schedule  # noqa: E402
from zenyx_b200.train import checkpoint as ckpt  # noqa: E402


def batches(vocab, batch, seq, seed=0):
    gen = torch.Generator().manual_seed(seed)
    while True:
        x = torch.randint(0, vocab, (batch, seq), generator=gen)
        yield x, torch.roll(x, -1, dims=1)


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=12)
    ap.add_argument("--dir", default="/tmp/zx_example02")
    args = ap.parse_args(argv)
    cfg = LlamaConfig.tiny(n_layers=2, d_model=256, n_heads=2, n_kv_heads=1, ffn_dim=512, vocab_size=512)
    seq, batch = 256, 2

    def make_trainer():
        sched = lr_schedule.warmup_cosine(2e-3, warmup_steps=3, total_steps=args.steps, min_lr=2e-4)
        return Trainer(cfg, TrainerConfig(lr=2e-3, seq_len=seq, global_batch=batch, max_grad_norm=1.0, lr_schedule=sched))

    # 1. a "pre-trained" model on disk, in the flat name -> tensor layout every loader understands
    base = make_trainer()
    pre = Path(args.dir) / "pretrained"
    ckpt.save(str(pre), 0, base.model)
    base.close()
    # 2. load it into a fresh trainer and fine-tune the first half of the steps, checkpointing at the end
    tr = make_trainer()
    missing, unexpected = loader.load_into(tr.model, str(pre / "step_0" / "model.safetensors"), chunk_size=8)
    assert not missing and not unexpected
    run_dir = str(Path(args.dir) / "run")
    half = loop.run(tr, batches(cfg.vocab_size, batch, seq), cfg=loop.LoopConfig(steps=args.steps // 2, log_every=2,
                                                                                checkpoint_dir=run_dir))
    tr.close()
    # 3. a new process would do exactly this: same config, resume=True picks up the last checkpoint
    tr2 = make_trainer()
    rest = loop.run(tr2, batches(cfg.vocab_size, batch, seq, seed=1),
                    cfg=loop.LoopConfig(steps=args.steps, log_every=2, checkpoint_dir=run_dir, resume=True))
    tr2.close()
    print(f"first half: loss {half[0]['loss']:.3f} -> {half[-1]['loss']:.3f}; resumed at step {rest[0]['step']}, "
          f"ended at {rest[-1]['loss']:.3f}; latest checkpoint: step {ckpt.latest_step(run_dir)}")
    return half, rest


if __name__ == "__main__":
    main()
