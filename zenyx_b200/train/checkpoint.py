"""Checkpoint / resume.

The reference ships no checkpoint code (its ``zenyx/train/checkpoint.py`` was deleted,
ZENYX_2_0_DELIVERABLES.txt:190). The two conventions it leaves behind are honoured:

* a flat ``{parameter name: tensor}`` map, which is what ``load_state_dict_chunked`` consumes
  (zenyx/train/loading.py:11-30)  ->  ``<dir>/step_<N>/model.safetensors`` (unsharded, written by rank 0);
* the examples' ``torch.save({'model','optimizer','config','metrics'})`` dict
  (examples/03_expert_tpu_v5e8_training.py:206-218)  ->  ``export_pt``.

Optimizer state is sharded: ``optim_rank<r>of<W>.safetensors`` holds that rank's slice of the fp32
master remainder, m and v plus its shard bounds; ``rng_rank<r>of<W>.json`` that rank's CPU RNG state;
``meta.json`` carries step, config, curriculum state, rank 0's RNG state and metrics. Files are written under a temporary name and renamed; a ``latest``
file points at the last complete step. Resume is bit-exact at the same world size, and valid across
world-size changes (the shards are re-partitioned from the per-rank files).
"""
from __future__ import annotations

import json
import os
from typing import Any, Dict, Optional

import torch
import torch.distributed as dist
from safetensors.torch import load_file, save_file


def _rank_world():
    if dist.is_available() and dist.is_initialized():
        return dist.get_rank(), dist.get_world_size()
    return 0, 1


def _atomic_write_bytes(path: str, data: bytes) -> None:
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(data)
        f.flush()
        os.fsync(f.fileno())
    os.replace(tmp, path)


def _atomic_save_tensors(path: str, tensors: Dict[str, torch.Tensor], metadata: Optional[Dict[str, str]] = None) -> None:
    tmp = path + ".tmp"
    save_file({k: v.detach().contiguous().cpu() for k, v in tensors.items()}, tmp, metadata=metadata)
    os.replace(tmp, path)


def model_state(model) -> Dict[str, torch.Tensor]:
    if hasattr(model, "state_dict_flat"):
        return model.state_dict_flat()
    return {k: v for k, v in model.state_dict().items()}


def save(ckpt_dir: str, step: int, model, optimizer=None, scheduler_state: Optional[Dict[str, Any]] = None,
         config: Optional[Dict[str, Any]] = None, metrics: Optional[Dict[str, Any]] = None) -> str:
    """Writes ``<ckpt_dir>/step_<step>/`` synchronously. Every rank writes its optimizer shard and its own
    RNG state; rank 0 writes the model, the metadata and, last, the ``latest`` pointer. Returns the step
    directory."""
    rank, world = _rank_world()
    d = os.path.join(ckpt_dir, f"step_{step}")
    os.makedirs(d, exist_ok=True)

    if optimizer is not None and hasattr(optimizer, "state_dict") and hasattr(optimizer, "n_shard"):
        sd = optimizer.state_dict()
        _atomic_save_tensors(os.path.join(d, f"optim_rank{rank}of{world}.safetensors"),
                             {"p_lo": sd["p_lo"], "m": sd["m"], "v": sd["v"]},
                             {"step": str(sd["step"]), "shard_begin": str(sd["shard_begin"]),
                              "n_shard": str(sd["n_shard"]), "world": str(world)})
    elif optimizer is not None and rank == 0:
        torch.save(optimizer.state_dict(), os.path.join(d, "optimizer.pt"))
    if rank == 0:
        _atomic_save_tensors(os.path.join(d, "model.safetensors"), model_state(model))
        meta = {"step": step, "world_size": world, "config": config or {}, "metrics": metrics or {},
                "scheduler": scheduler_state or {}, "torch_rng": torch.get_rng_state().tolist()}
        _atomic_write_bytes(os.path.join(d, "meta.json"), json.dumps(meta, default=str).encode())

    _atomic_write_bytes(os.path.join(d, f"rng_rank{rank}of{world}.json"),
                        json.dumps({"torch_rng": torch.get_rng_state().tolist()}).encode())
    if world > 1:
        dist.barrier()
    if rank == 0:
        _atomic_write_bytes(os.path.join(ckpt_dir, "latest"), str(step).encode())
    return d


def latest_step(ckpt_dir: str) -> Optional[int]:
    p = os.path.join(ckpt_dir, "latest")
    if not os.path.exists(p):
        return None
    return int(open(p).read().strip())


def load(ckpt_dir: str, model, optimizer=None, step: Optional[int] = None, strict: bool = True) -> Dict[str, Any]:
    """Restores model (and optimizer) in place; returns the metadata dict."""
    from .loading import load_state_dict_chunked

    rank, world = _rank_world()
    step = latest_step(ckpt_dir) if step is None else step
    if step is None:
        raise FileNotFoundError(f"no checkpoint under {ckpt_dir}")
    d = os.path.join(ckpt_dir, f"step_{step}")
    meta = json.loads(open(os.path.join(d, "meta.json")).read())
    load_state_dict_chunked(model, load_file(os.path.join(d, "model.safetensors")), strict=strict)
    if optimizer is not None and hasattr(optimizer, "n_shard"):
        saved_world = int(meta["world_size"])
        own = os.path.join(d, f"optim_rank{rank}of{world}.safetensors")
        if saved_world == world and os.path.exists(own):
            t = load_file(own)
            optimizer.load_state_dict({"step": step_of(own), "shard_begin": optimizer.shard_begin,
                                       "n_shard": optimizer.n_shard, "p_lo": t["p_lo"], "m": t["m"], "v": t["v"]})
        else:  # re-partition: stitch the saved shards together, then slice
            parts = [load_file(os.path.join(d, f"optim_rank{r}of{saved_world}.safetensors")) for r in range(saved_world)]
            full = {k: torch.cat([p[k] for p in parts]) for k in ("p_lo", "m", "v")}
            optimizer.load_full_state(step_of(os.path.join(d, f"optim_rank0of{saved_world}.safetensors")),
                                      full["p_lo"], full["m"], full["v"])
    elif optimizer is not None and os.path.exists(os.path.join(d, "optimizer.pt")):
        optimizer.load_state_dict(torch.load(os.path.join(d, "optimizer.pt"), map_location="cpu"))
    own_rng = os.path.join(d, f"rng_rank{rank}of{world}.json")
    if os.path.exists(own_rng):      # same world size: every rank continues its own random stream
        torch.set_rng_state(torch.tensor(json.loads(open(own_rng).read())["torch_rng"], dtype=torch.uint8))
    elif "torch_rng" in meta:        # re-partitioned run: rank 0's stream is the only common reference
        torch.set_rng_state(torch.tensor(meta["torch_rng"], dtype=torch.uint8))
    return meta


def step_of(optim_file: str) -> int:
    from safetensors import safe_open

    with safe_open(optim_file, framework="pt") as f:
        return int(f.metadata()["step"])


def export_pt(path: str, model, optimizer=None, config: Optional[Dict[str, Any]] = None,
              metrics: Optional[Dict[str, Any]] = None) -> None:
    """The single-file layout of the reference's examples: {'model','optimizer','config','metrics'}."""
    opt_sd = None
    if optimizer is not None:
        sd = optimizer.state_dict()
        opt_sd = {k: (v.cpu() if isinstance(v, torch.Tensor) else v) for k, v in sd.items()}
    torch.save({"model": {k: v.detach().cpu() for k, v in model_state(model).items()}, "optimizer": opt_sd,
                "config": config or {}, "metrics": metrics or {}}, path)
