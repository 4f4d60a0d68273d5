"""Multi-rank host logic on CPU: gloo process groups, world size 2 (spawned processes)."""
import math
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp
import torch.nn as nn


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _entry(rank, world, port, fn, args):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    torch.manual_seed(0)
    torch.set_num_threads(2)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        fn(rank, world, *args)
    finally:
        dist.destroy_process_group()


def run_ranks(fn, world=2, args=()):
    mp.spawn(_entry, args=(world, _free_port(), fn, args), nprocs=world, join=True)


# ------------------------------------------------------------------------------------------------
def _ring_attention(rank, world):
    from zenyx_b200.ops.attention import (MaskSpec, RingContext, attn_backward, attn_forward, ring_attn_backward,
                                          ring_attn_forward, shard_sequence)

    B, S, Hq, Hkv, D = 1, 256 * world, 2, 1, 128
    g = torch.Generator().manual_seed(3)
    q, k, v, do = (torch.randn(B, S, h, D, generator=g) for h in (Hq, Hkv, Hkv, Hq))
    scale = 1 / math.sqrt(D)
    for mask in (MaskSpec(True), MaskSpec(True, 1, 2)):
        o_ref, lse_ref = torch.empty_like(q), torch.empty(B, Hq, S)
        attn_forward(q, k, v, o_ref, lse_ref, scale, mask, [0], [0])
        dq_ref, dk_ref, dv_ref = torch.empty_like(q), torch.zeros_like(k), torch.zeros_like(v)
        attn_backward(q, k, v, o_ref, do, lse_ref, torch.empty_like(lse_ref), dq_ref, dk_ref, dv_ref, scale, mask, [0], [0])
        ring = RingContext(rank=rank, degree=world, seq_len=S, mask=mask)
        sh = lambda t, dim=1: shard_sequence(t, rank, world, dim=dim).contiguous()
        o, lse = ring_attn_forward(ring, sh(q), sh(k), sh(v), scale)
        dq, dk, dv = ring_attn_backward(ring, sh(q), sh(k), sh(v), o, sh(do), lse, scale)
        assert torch.allclose(o, sh(o_ref), atol=1e-5) and torch.allclose(lse, sh(lse_ref, 2), atol=1e-5)
        assert torch.allclose(dq, sh(dq_ref), atol=1e-4) and torch.allclose(dk, sh(dk_ref), atol=1e-4)
        assert torch.allclose(dv, sh(dv_ref), atol=1e-4)


@pytest.mark.parametrize("world", [2, 3, 4])
def test_ring_attention_schedule_matches_full_attention(world):
    run_ranks(_ring_attention, world=world)


# ------------------------------------------------------------------------------------------------
def _zero_and_engine(rank, world):
    from zenyx_b200.models import LlamaConfig, LlamaModel
    from zenyx_b200.parallel.zero import ZeroAdamW
    from zenyx_b200.train import Trainer, TrainerConfig

    cfg = LlamaConfig.tiny(n_layers=1, d_model=64, n_heads=2, n_kv_heads=1, ffn_dim=96, vocab_size=128)
    S = 256 * world
    g = torch.Generator().manual_seed(9)
    tok = torch.randint(0, 128, (world, S), generator=g)
    # single-process reference: the whole global batch on one model
    ref = LlamaModel(cfg, seed=4)
    ropt = ZeroAdamW(ref.flat, lr=1e-2, max_grad_norm=1.0, weight_decay=0.1, single_process=True)
    ref_losses = []
    for _ in range(3):
        loss = sum(ref.forward_backward(tok[i:i + 1], tok[i:i + 1], 1.0 / (world * S)) for i in range(world))
        ropt.step()
        ref_losses.append(float(loss))
    for cp in (world, 1):
        tr = Trainer(cfg, TrainerConfig(lr=1e-2, seq_len=S, global_batch=world, ring_degree=cp, max_grad_norm=1.0,
                                        weight_decay=0.1, seed=4))
        losses = [tr.train_step(tok, tok) for _ in range(3)]
        assert all(abs(a - b) < 2e-2 for a, b in zip(losses, ref_losses)), (cp, losses, ref_losses)
        # parameters identical on every rank after the sharded update + all-gather
        p = tr.model.flat.params.float()
        q = p.clone()
        dist.broadcast(q, 0)
        assert torch.equal(p, q)
        for name in ("layers.0.wqkv", "lm_head.weight", "final_norm"):
            a, b = tr.model.w(name).float(), ref.w(name).float()
            assert (a - b).norm() / b.norm() < 2e-2, (cp, name)


def test_sharded_optimizer_and_dp_cp_training_match_single_process():
    run_ranks(_zero_and_engine)


# ------------------------------------------------------------------------------------------------
def _tensor_parallel(rank, world):
    from zenyx_b200.distributed import (ColumnParallelLinear, RowParallelLinear, TensorParallelEmbedding,
                                        make_tensor_parallel_model)

    torch.manual_seed(1)
    full = nn.Sequential(nn.Embedding(32, 16), nn.Linear(16, 24), nn.GELU(), nn.Linear(24, 8), nn.Linear(8, 6))
    ids = torch.randint(0, 32, (5, 7))
    ref = full(ids)
    ref.sum().backward()
    ref_grads = {n: p.grad.clone() for n, p in full.named_parameters()}
    import copy

    tp = make_tensor_parallel_model(copy.deepcopy(full).requires_grad_(True))
    for p in tp.parameters():
        p.grad = None
    assert isinstance(tp[0], TensorParallelEmbedding) and isinstance(tp[1], ColumnParallelLinear)
    assert isinstance(tp[3], RowParallelLinear) and isinstance(tp[4], ColumnParallelLinear)
    out = tp(ids)
    assert out.requires_grad and torch.allclose(out, ref, atol=1e-5)
    out.sum().backward()
    n1 = tp[1].local_out
    assert torch.allclose(tp[1].weight.grad, ref_grads["1.weight"][rank * n1:(rank + 1) * n1], atol=1e-5)
    n3 = tp[3].local_in
    assert torch.allclose(tp[3].weight.grad, ref_grads["3.weight"][:, rank * n3:(rank + 1) * n3], atol=1e-5)
    assert torch.allclose(tp[3].bias.grad, ref_grads["3.bias"], atol=1e-5)
    nv = tp[0].local_vocab
    assert torch.allclose(tp[0].weight.grad, ref_grads["0.weight"][rank * nv:(rank + 1) * nv], atol=1e-5)


def test_tensor_parallel_layers_forward_and_backward():
    run_ranks(_tensor_parallel)


# ------------------------------------------------------------------------------------------------
def _sequence_parallel_linears(rank, world):
    """all-gather -> GEMM and GEMM -> reduce-scatter (host fallbacks of the fused kernels) and the
    two sequence-parallel layers: forward and every gradient against a single-process MLP."""
    from zenyx_b200.distributed import SequenceParallelColumnLinear, SequenceParallelRowLinear
    from zenyx_b200.parallel.fused_collective import allgather_gemm, gemm_reduce_scatter

    torch.manual_seed(5)
    m, K, H, N = 6, 8, 12, 8
    x_all = torch.randn(world * m, K)
    w1, w2 = torch.randn(H, K) / 3, torch.randn(N, H) / 3
    y = allgather_gemm(x_all[rank * m:(rank + 1) * m], w1)
    assert torch.allclose(y, x_all @ w1.t(), atol=1e-5)
    kl = K // world
    yr = gemm_reduce_scatter(x_all[:, rank * kl:(rank + 1) * kl].contiguous(), w1[:, rank * kl:(rank + 1) * kl].contiguous())
    assert torch.allclose(yr, (x_all @ w1.t())[rank * m:(rank + 1) * m], atol=1e-5)
    # column (token-sharded input) -> tanh -> row (token-sharded output)
    xr = x_all.clone().requires_grad_(True)
    ref = torch.tanh(xr @ w1.t()) @ w2.t()
    ref.square().sum().backward()
    hl = H // world
    col = SequenceParallelColumnLinear(K, H, dtype=torch.float32)
    row = SequenceParallelRowLinear(H, N, dtype=torch.float32)
    with torch.no_grad():
        col.weight.copy_(w1[rank * hl:(rank + 1) * hl])
        row.weight.copy_(w2[:, rank * hl:(rank + 1) * hl])
    xl = x_all[rank * m:(rank + 1) * m].clone().requires_grad_(True)
    out = row(torch.tanh(col(xl)))
    assert torch.allclose(out, ref[rank * m:(rank + 1) * m].detach(), atol=1e-5)
    out.square().sum().backward()
    assert torch.allclose(xl.grad, xr.grad[rank * m:(rank + 1) * m], atol=1e-4)
    w1r, w2r = w1.clone().requires_grad_(True), w2.clone().requires_grad_(True)
    (torch.tanh(x_all @ w1r.t()) @ w2r.t()).square().sum().backward()
    assert torch.allclose(col.weight.grad, w1r.grad[rank * hl:(rank + 1) * hl], atol=1e-4)
    assert torch.allclose(row.weight.grad, w2r.grad[:, rank * hl:(rank + 1) * hl], atol=1e-4)


def test_sequence_parallel_linears_match_single_process():
    run_ranks(_sequence_parallel_linears)


# ------------------------------------------------------------------------------------------------
def _ring_helpers_and_vocab_ce(rank, world):
    from zenyx_b200.ops.comm import ring_all_gather, ring_exchange, ring_reduce_scatter
    from zenyx_b200.ops.vocab import vocab_parallel_cross_entropy

    x = torch.full((3,), float(rank))
    got = ring_exchange(x)
    assert torch.equal(got, torch.full((3,), float((rank - 1) % world)))
    parts = ring_all_gather(x)
    assert all(torch.equal(parts[r], torch.full((3,), float(r))) for r in range(world))
    contrib = [torch.full((2,), float(10 * rank + o)) for o in range(world)]       # my share for owner o
    mine = ring_reduce_scatter(contrib)
    assert torch.allclose(mine, torch.full((2,), float(sum(10 * q + rank for q in range(world)))))
    # vocabulary-parallel cross-entropy against the unsharded loss and gradient
    torch.manual_seed(3)
    T, V = 9, 8 * world
    logits = torch.randn(T, V, requires_grad=True)
    tgt = torch.randint(0, V, (T,))
    ref = torch.nn.functional.cross_entropy(logits, tgt, reduction="none")
    ref.sum().backward()
    vl = V // world
    local = logits.detach()[:, rank * vl:(rank + 1) * vl].clone().requires_grad_(True)
    loss = vocab_parallel_cross_entropy(local, tgt)
    assert torch.allclose(loss, ref.detach(), atol=1e-5)
    loss.sum().backward()
    assert torch.allclose(local.grad, logits.grad[:, rank * vl:(rank + 1) * vl], atol=1e-5)


@pytest.mark.parametrize("world", [2, 3, 4])
def test_ring_helpers_and_vocab_parallel_cross_entropy(world):
    run_ranks(_ring_helpers_and_vocab_ce, world=world)


# ------------------------------------------------------------------------------------------------
def _pipeline(rank, world, schedule):
    from zenyx_b200.distributed import DistributedPipelineEngine, PipelineParallelModel

    torch.manual_seed(2)
    layers = [nn.Linear(8, 16), nn.Tanh(), nn.Linear(16, 16), nn.Tanh(), nn.Linear(16, 4)]
    full = nn.Sequential(*layers)
    import copy

    single = copy.deepcopy(full)
    x, y = torch.randn(8, 8), torch.randn(8, 4)
    sopt = torch.optim.SGD(single.parameters(), lr=0.1)
    ref_losses = []
    for _ in range(2):
        sopt.zero_grad()
        l = nn.functional.mse_loss(single(x), y)
        l.backward()
        sopt.step()
        ref_losses.append(float(l))
    ppm = PipelineParallelModel(copy.deepcopy(full), num_stages=world, stage_id=rank)
    opt = torch.optim.SGD(ppm.stage.parameters(), lr=0.1)
    mb_shape = (2, 8) if rank == 0 else (2, 16)
    eng = DistributedPipelineEngine(ppm.stage, opt, loss_fn=nn.functional.mse_loss, micro_batch_shape=mb_shape,
                                    num_microbatches=4, schedule=schedule)
    for step in range(2):
        loss = eng.run_step(x if rank == 0 else None, y if rank == world - 1 else None)
        if rank == world - 1:
            assert abs(loss - ref_losses[step]) < 1e-5, (loss, ref_losses[step])
    mine = list(ppm.stage.parameters())
    ref_params = list(single.parameters())
    offset = 0 if rank == 0 else len(ref_params) - len(mine)
    for a, b in zip(mine, ref_params[offset: offset + len(mine)]):
        assert torch.allclose(a, b, atol=1e-5)


@pytest.mark.parametrize("schedule", ["1f1b", "gpipe"])
def test_pipeline_engine_matches_single_process(schedule):
    run_ranks(_pipeline, args=(schedule,))


def test_single_process_schedules_agree():
    from zenyx_b200.distributed import Partial1F1BSchedule, SimpleGPipeSchedule, create_pipeline_from_sequential
    from zenyx_b200.parallel.pipeline_parallel import one_f_one_b_order

    torch.manual_seed(3)
    model = nn.Sequential(nn.Linear(4, 8), nn.ReLU(), nn.Linear(8, 8), nn.ReLU(), nn.Linear(8, 2))
    stages = create_pipeline_from_sequential(model, 3)
    assert [len(s.layers) for s in stages] == [2, 2, 1]
    x, y = torch.randn(8, 4), torch.randn(8, 2)
    a = SimpleGPipeSchedule(stages, 4).step(x, y, nn.functional.mse_loss)
    g1 = [p.grad.clone() for p in model.parameters()]
    model.zero_grad()
    b = Partial1F1BSchedule(stages, 4).step(x, y, nn.functional.mse_loss)
    assert abs(a - b) < 1e-6
    for u, v in zip(g1, model.parameters()):
        assert torch.allclose(u, v.grad, atol=1e-6)
    order = one_f_one_b_order(0, 4, 8)
    assert order[:3] == [("F", 0), ("F", 1), ("F", 2)] and order[3:5] == [("F", 3), ("B", 0)]
    assert sorted(i for op, i in order if op == "B") == list(range(8))


# ------------------------------------------------------------------------------------------------
def _collectives_and_reducer(rank, world):
    from zenyx_b200.distributed import CollectiveGroup, all_gather, all_reduce, broadcast, reduce_scatter
    from zenyx_b200.runtime import Scheduler

    t = torch.full((4, 6), float(rank + 1))
    nc = t.t()                                   # non-contiguous view is still updated in place
    all_reduce(nc, op="sum")
    assert torch.all(t == 3.0)
    h = all_reduce(torch.ones(3) * rank, op="max", async_op=True)
    assert torch.all(h.wait() == 1.0) and h.is_completed()
    b = torch.arange(4.0) * (rank + 1)
    broadcast(b, src=1)
    assert torch.equal(b, torch.arange(4.0) * 2)
    out = torch.empty(2 * 3)
    all_gather(out, torch.full((3,), float(rank)))
    assert out.tolist() == [0, 0, 0, 1, 1, 1]
    assert CollectiveGroup().world_size == 2
    with pytest.raises(ValueError):
        all_reduce(torch.ones(1), op="median")
    # data-parallel scheduler: gradients averaged once per optimizer step, replicas stay identical
    torch.manual_seed(0)
    model = nn.Sequential(nn.Linear(8, 8), nn.ReLU(), nn.Linear(8, 2))
    opt = torch.optim.SGD(model.parameters(), lr=0.1)
    sched = Scheduler(accumulation_steps=2, enable_overlap=False, bucket_size_mb=0.0001)
    g = torch.Generator().manual_seed(100 + rank)
    for _ in range(4):
        x, y = torch.randn(4, 8, generator=g), torch.randn(4, 2, generator=g)
        sched.backward(nn.functional.mse_loss(model(x), y), model=model, optimizer=opt)
    assert sched.step_count == 2
    for p in model.parameters():
        q = p.detach().clone()
        dist.broadcast(q, 0)
        assert torch.equal(p.detach(), q)


def test_collectives_and_bucket_reducer():
    run_ranks(_collectives_and_reducer)


# ------------------------------------------------------------------------------------------------
def _failure_detection(rank, world):
    import time

    from zenyx_b200.core import FaultInjector, Heartbeat, RankFailure

    hb = Heartbeat.from_process_group(timeout_s=0.6)
    inj = FaultInjector("2:1:stall", rank=rank)
    detected = False
    for step in range(40):
        hb.beat(step)
        inj.maybe_fail(step, hb)                 # rank 1 stops beating from step 2 on (host-side only)
        time.sleep(0.05)
        if rank == 0:
            try:
                hb.check()
            except RankFailure:
                detected = True
                break
    if rank == 0:
        assert detected, "rank 0 never noticed that rank 1 stopped reporting"
    with pytest.raises(RankFailure):
        FaultInjector("5:%d:raise" % rank, rank=rank).maybe_fail(5)
    with pytest.raises(ValueError):
        FaultInjector("1:0:explode")


def test_heartbeat_detects_a_stalled_rank_on_the_host():
    run_ranks(_failure_detection)


# ------------------------------------------------------------------------------------------------
def _elastic(rank, world, tmp):
    """Three data-parallel gloo ranks train a tiny Llama; rank 2 leaves between steps (host-side exit, nothing in
    flight); the other two notice, agree on the roster, form a 2-rank group, resume from the last checkpoint
    (sharded optimizer state re-sharded 3 -> 2) and finish the run."""
    from zenyx_b200.models import LlamaConfig
    from zenyx_b200.train import Trainer, TrainerConfig, loop
    from zenyx_b200.train import checkpoint as ckpt
    from zenyx_b200.train.elastic import ElasticConfig, run_elastic

    cfg = LlamaConfig.tiny(n_layers=1, d_model=64, n_heads=2, n_kv_heads=1, ffn_dim=96, vocab_size=128)
    seq, batch, steps = 128, 6, 6

    def make_trainer():
        return Trainer(cfg, TrainerConfig(lr=5e-3, seq_len=seq, global_batch=batch, ring_degree=1, max_grad_norm=1.0, seed=1))

    def make_data(r, w):
        gen = torch.Generator().manual_seed(7)
        while True:
            x = torch.randint(0, 128, (batch, seq), generator=gen)
            yield x, torch.roll(x, -1, dims=1)

    def fault(step):
        if rank == 2 and step == 3:
            os._exit(0)          # leaves between steps, the way a crashed host process would

    records, coord = run_elastic(make_trainer, make_data,
                                 loop.LoopConfig(steps=steps, log_every=0, checkpoint_every=2,
                                                 checkpoint_dir=os.path.join(tmp, "ckpt"), resume=True),
                                 ElasticConfig(rendezvous_dir=os.path.join(tmp, "rdzv"), heartbeat_timeout_s=2.0,
                                               settle_s=1.0, group_timeout_s=60.0), before_step=fault)
    assert coord.generation == 1 and dist.get_world_size() == 2 and dist.get_rank() == rank
    assert records[0]["step"] == 2 and records[-1]["step"] == steps - 1      # resumed from the step-2 checkpoint
    assert all(math.isfinite(r["loss"]) for r in records)
    assert ckpt.latest_step(os.path.join(tmp, "ckpt")) == steps


def test_elastic_regroup_after_a_rank_leaves(tmp_path):
    run_ranks(_elastic, world=3, args=(str(tmp_path),))
