"""``bench.py --impl reference``: the same metric and configuration measured on the UNMODIFIED
reference package (``baseline/_ref/zenyx``), through its own public API and stock code path:

* ``zenyx.train.Trainer(model, TrainerConfig(lr, accumulation_steps))``  (zenyx/train/trainer.py:16-57)
  -> ``Scheduler.forward/backward`` + ``GradientBucketReducer`` all-reduce + ``torch.optim.AdamW``;
* ``zenyx.memory.ActivationManager`` for activation checkpointing (zenyx/memory/activation_manager.py).

The reference has neither a Llama model nor ring attention, so the model is the stock-PyTorch
``baseline/torch_llama.TorchLlama`` (bf16 parameters, cuBLAS + SDPA), and more than one GPU means
the reference's only strategy that runs this model: data parallelism over whole sequences
(global batch 8 = N ranks x 8/N accumulated micro-batches of one 32K sequence).
Nothing from ``zenyx_b200`` is imported on this path.
"""
from __future__ import annotations

import json
import os
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")


def unavailable(why: str) -> None:
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)


def run_reference(args) -> None:
    if not os.path.isdir(os.path.join(REF, "zenyx")):
        unavailable("reference package is not installed under baseline/_ref")
        return
    sys.path.insert(0, REF)
    try:
        import torch
        import torch.distributed as dist
        import zenyx  # noqa: F401  (the reference)
        from zenyx.memory import ActivationManager, CheckpointPolicy
        from zenyx.train import Trainer, TrainerConfig
    except Exception as e:  # noqa: BLE001
        unavailable(f"cannot import the reference: {type(e).__name__}: {e}"[:300])
        return
    sys.path.insert(0, os.path.dirname(HERE))
    from baseline.torch_llama import TokenCrossEntropy, TorchLlama
    from bench import ClockSampler

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    if not torch.cuda.is_available():
        unavailable("no CUDA device")
        return
    B, S = args.global_batch, args.seq_len
    if B % world != 0:
        unavailable(f"global batch {B} does not split over {world} data-parallel ranks")
        return
    accum = B // world
    try:
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
        torch.manual_seed(0)
        with torch.device("cuda"):
            model = TorchLlama(n_layers=args.layers).to(torch.bfloat16)
        ActivationManager(CheckpointPolicy(checkpoint_attention=True, checkpoint_ffn=True)).hook_into_model(model)
        trainer = Trainer(model, TrainerConfig(lr=3e-4, accumulation_steps=accum))
        criterion = TokenCrossEntropy()
        dev = trainer.ctx.device
        vocab = 128256
        n_steps = args.warmup + 2 * args.steps
        gen = torch.Generator().manual_seed(1234 + rank)
        toks = [[torch.randint(0, vocab, (1, S), generator=gen).pin_memory() for _ in range(accum)] for _ in range(n_steps)]
        tgts = [[torch.randint(0, vocab, (1, S), generator=gen).pin_memory() for _ in range(accum)] for _ in range(n_steps)]

        def sync_all():
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()

        def max_over_ranks(ms):
            t = torch.tensor([ms], device=dev, dtype=torch.float64)
            if world > 1:
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t.item())

        def one_step(i, on_device=False):
            last = 0.0
            for j in range(accum):
                x, y = toks[i][j], tgts[i][j]
                if on_device:
                    x, y = x.to(dev), y.to(dev)
                last = trainer.train_step(x, y, criterion)
            return last

        for i in range(args.warmup):
            one_step(i)
        sampler = ClockSampler(torch.cuda.current_device())
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        dev_batches = [([t.to(dev) for t in toks[args.warmup + i]], [t.to(dev) for t in tgts[args.warmup + i]])
                       for i in range(args.steps)]
        sync_all()
        sampler.start()
        e0.record()
        for xs, ys in dev_batches:
            for x, y in zip(xs, ys):
                trainer.train_step(x, y, criterion)
        e1.record()
        sync_all()
        clocks = sampler.stop()
        ms_dev = max_over_ranks(e0.elapsed_time(e1))
        del dev_batches
        base = args.warmup + args.steps
        sync_all()
        t0 = time.perf_counter()
        e0.record()
        last = 0.0
        for i in range(args.steps):
            last = one_step(base + i)
        e1.record()
        sync_all()
        ms_e2e = max(max_over_ranks(e0.elapsed_time(e1)), max_over_ranks((time.perf_counter() - t0) * 1e3))
    except torch.cuda.OutOfMemoryError as e:
        unavailable(f"the reference stack runs out of device memory on this configuration: {str(e)[:160]}")
        return
    except Exception as e:  # noqa: BLE001
        unavailable(f"the reference stack failed: {type(e).__name__}: {str(e)[:200]}")
        return
    valid_shape = args.layers == 32 and S == 32768 and B == 8
    out = {
        "metric": "8B-shape 32K-ctx train tokens/s", "value": round(B * S * args.steps / (ms_dev / 1e3), 1),
        "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms_dev / args.steps, 2), "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "reference",
        "config": {"model": "llama3-8b-shape" + ("" if valid_shape else f"-DEBUG-{args.layers}L"), "global_batch": B,
                   "seq_len": S, "parallelism": f"dp{world}",
                   "stack": "reference Trainer/Scheduler/GradientBucketReducer + torch AdamW, stock PyTorch model "
                            "(cuBLAS, SDPA), reference ActivationManager checkpointing",
                   "l2": "inputs larger than L2"},
        "clocks": clocks,
        "e2e": {"value": round(B * S * args.steps / (ms_e2e / 1e3), 1), "unit": "tokens/s",
                "h2d_bytes_per_step": 2 * accum * S * 8, "d2h_bytes_per_step": 4 * accum, "last_loss": round(float(last), 4)},
        "gpu_launches": 0,
    }
    if rank == 0:
        print(json.dumps(out), flush=True)
    if world > 1 and dist.is_initialized():
        dist.destroy_process_group()
