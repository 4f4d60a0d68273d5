"""``bench.py --impl reference``: the same metric and configuration measured on the UNMODIFIED
reference package (``baseline/_ref/zenyx``), through its own public API and stock code path:

* ``zenyx.train.Trainer(model, TrainerConfig(lr, accumulation_steps))``  (zenyx/train/trainer.py:16-57)
  -> ``Scheduler.forward/backward`` + ``GradientBucketReducer`` all-reduce + ``torch.optim.AdamW``;
* ``zenyx.memory.ActivationManager.hook_into_model`` with the reference's default ``CheckpointPolicy()``
  (MLP blocks checkpointed, attention not; zenyx/memory/activation_manager.py:16-20,53-72). Only if that runs out
  of device memory the arm retries with attention checkpointed as well and says so in ``config.stack``.

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
    from bench import ClockSampler, workload_config

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
    vocab = 128256
    n_steps = args.warmup + args.steps
    gen = torch.Generator().manual_seed(1234 + rank)
    toks = [[torch.randint(0, vocab, (1, S), generator=gen).pin_memory() for _ in range(accum)] for _ in range(n_steps)]
    tgts = [[torch.randint(0, vocab, (1, S), generator=gen).pin_memory() for _ in range(accum)] for _ in range(n_steps)]
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))

    def attempt(policy):
        """Builds the model under `policy`, runs warm-up + the timed steps, returns (ms_dev, ms_wall, clocks, loss)."""
        torch.manual_seed(0)
        with torch.device("cuda"):
            model = TorchLlama(n_layers=args.layers).to(torch.bfloat16)
        ActivationManager.hook_into_model(model, use_checkpoint=True, policy=policy)
        trainer = Trainer(model, TrainerConfig(lr=3e-4, accumulation_steps=accum))
        criterion = TokenCrossEntropy()
        dev = trainer.ctx.device

        def sync_all():
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()

        def max_over_ranks(ms):
            t = torch.tensor([ms], device=dev, dtype=torch.float64)
            if world > 1:
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t.item())

        def one_step(i):   # pinned host tokens in, host float loss out, through the reference Trainer
            last = 0.0
            for j in range(accum):
                last = trainer.train_step(toks[i][j], tgts[i][j], criterion)
            return last

        for i in range(args.warmup):
            one_step(i)
        sampler = ClockSampler(torch.cuda.current_device())
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        sync_all()
        sampler.start()
        t0 = time.perf_counter()
        e0.record()
        last = 0.0
        for i in range(args.steps):
            last = one_step(args.warmup + i)
        e1.record()
        sync_all()
        wall = (time.perf_counter() - t0) * 1e3
        clocks = sampler.stop()
        return max_over_ranks(e0.elapsed_time(e1)), max_over_ranks(wall), clocks, last

    policy_note = "reference default CheckpointPolicy (MLP checkpointed, attention kept)"
    try:
        result = None
        try:
            result = attempt(CheckpointPolicy())
        except torch.cuda.OutOfMemoryError:
            pass   # retried below, outside the handler, so that the failed attempt's frames (model, trainer) are gone
        if result is None:
            # every rank runs the same model on the same shapes, so all of them land here together
            import gc

            gc.collect()
            torch.cuda.empty_cache()
            policy_note = "CheckpointPolicy(checkpoint_attention=True) after the default ran out of memory"
            result = attempt(CheckpointPolicy(checkpoint_attention=True, checkpoint_ffn=True))
        ms_dev, ms_e2e, clocks, last = result
    except torch.cuda.OutOfMemoryError as e:
        unavailable(f"the reference stack runs out of device memory on this configuration: {str(e)[:160]}")
        return
    except Exception as e:  # noqa: BLE001
        unavailable(f"the reference stack failed: {type(e).__name__}: {str(e)[:200]}")
        return
    out = {
        "metric": "8B-shape 32K-ctx train tokens/s", "value": round(B * S * args.steps / (ms_dev / 1e3), 1),
        "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms_dev / args.steps, 2), "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "reference",
        "config": workload_config(args, f"dp{world}",
                                  "reference Trainer/Scheduler/GradientBucketReducer + torch AdamW (bf16 state), stock "
                                  "PyTorch model (cuBLAS, SDPA), " + policy_note),
        "clocks": clocks,
        "e2e": {"value": round(B * S * args.steps / (ms_e2e / 1e3), 1), "unit": "tokens/s",
                "h2d_bytes_per_step": 2 * accum * S * 8, "d2h_bytes_per_step": 4 * accum, "last_loss": round(float(last), 4)},
        "gpu_launches": 0,
    }
    if rank == 0:
        print(json.dumps(out), flush=True)
    if world > 1 and dist.is_initialized():
        dist.destroy_process_group()
