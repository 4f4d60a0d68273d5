import pytest
import torch
import torch.nn as nn

from zenyx_b200.memory import ActivationManager, CheckpointPolicy, MemoryTracker
from zenyx_b200.runtime import (ExecutionGraph, ExecutionGraphBuilder, ExecutionPlan, OpNode, OpType, Scheduler,
                                TopologyConfig, validate_graph)


def _mlp():
    return nn.Sequential(nn.Linear(8, 16), nn.ReLU(), nn.Linear(16, 4))


def test_graph_rejects_duplicates_unknowns_and_cycles():
    g = ExecutionGraph()
    g.add_node(OpNode("a", OpType.FORWARD))
    g.add_node(OpNode("b", OpType.FORWARD))
    g.add_node(OpNode("c", OpType.BACKWARD))
    with pytest.raises(ValueError):
        g.add_node(OpNode("a", OpType.FORWARD))
    with pytest.raises(ValueError):
        g.add_dependency("a", "zzz")
    g.add_dependency("b", "a")
    g.add_dependency("c", "b")
    with pytest.raises(ValueError):
        g.add_dependency("a", "c")
    assert g.topological_order() == ["a", "b", "c"]
    assert g.get_forward_execution_order() == ["a", "b"] and g.get_backward_execution_order() == ["c"]
    assert g.validate()


def test_builder_output_validates_and_executes():
    model = _mlp()
    g = ExecutionGraphBuilder().build_from_model(model, torch.randn(2, 8), world_size=2)
    res = validate_graph(g)
    assert res.is_valid, res.errors
    s = g.summarize()
    assert s["num_forward"] == 3 and s["num_backward"] == 3 and s["num_comm"] == 1 and s["total_params"] == 212
    assert s["total_flops"] > 0
    sched = Scheduler(enable_overlap=False)
    opt = torch.optim.SGD(model.parameters(), lr=0.1)
    loss = model(torch.randn(2, 8)).pow(2).mean()
    sched.backward(loss, model=model, optimizer=opt, execution_graph=g)   # single process: all-reduce is a no-op
    assert sched.step_count == 1


def test_validator_reports_deadlock_and_missing_tensor():
    g = ExecutionGraph()
    g.add_node(OpNode("x", OpType.FORWARD))
    g.add_node(OpNode("y", OpType.FORWARD))
    g.add_node(OpNode("ar", OpType.ALLREDUCE, metadata={"op": "bogus"}))
    g.dependencies["x"].append("y")
    g.dependents["y"].append("x")
    g.dependencies["y"].append("x")
    g.dependents["x"].append("y")
    res = validate_graph(g)
    assert not res.is_valid
    assert any("deadlock" in e for e in res.errors)
    assert any("metadata['tensor']" in e for e in res.errors)
    assert any("unknown reduce op" in e for e in res.errors)


def test_scheduler_priority_compute_then_intra_then_inter():
    g = ExecutionGraph()
    g.add_node(OpNode("inter", OpType.ALLREDUCE, device_ids=[0, 8], metadata={"tensor": torch.zeros(1)}))
    g.add_node(OpNode("intra", OpType.ALLREDUCE, device_ids=[0, 1], metadata={"tensor": torch.zeros(1)}))
    g.add_node(OpNode("comp", OpType.BACKWARD))
    s = Scheduler(enable_overlap=False, topology=TopologyConfig(intra_node_ranks=[0, 1, 2, 3], inter_node_ranks=[0, 8]))
    assert s._execute_graph_nodes(g) == ["comp", "intra", "inter"]


def test_accumulation_steps_once_and_scales_like_a_big_batch():
    torch.manual_seed(0)
    m1, m2 = _mlp(), _mlp()
    m2.load_state_dict(m1.state_dict())
    x, y = torch.randn(8, 8), torch.randn(8, 4)
    o1 = torch.optim.SGD(m1.parameters(), lr=0.1)
    o2 = torch.optim.SGD(m2.parameters(), lr=0.1)
    s = Scheduler(accumulation_steps=2, enable_overlap=False)
    for i in range(2):
        xb, yb = x[i * 4:(i + 1) * 4], y[i * 4:(i + 1) * 4]
        s.backward(nn.functional.mse_loss(m1(xb), yb), model=m1, optimizer=o1)
        assert s.step_count == i  # steps only at the boundary
    nn.functional.mse_loss(m2(x), y).backward()
    o2.step()
    for a, b in zip(m1.parameters(), m2.parameters()):
        assert torch.allclose(a, b, atol=1e-6)
    assert s.get_stats()["step"] == 1 and s.accumulated_loss > 0


def test_backward_accepts_quickstart_call_form():
    m = _mlp()
    opt = torch.optim.SGD(m.parameters(), lr=0.1)
    before = [p.clone() for p in m.parameters()]
    Scheduler(enable_overlap=False).backward(m(torch.randn(2, 8)).mean(), opt)
    assert any(not torch.equal(a, b) for a, b in zip(before, m.parameters()))


def test_activation_manager_selects_and_restores():
    class Block(nn.Module):
        def __init__(self):
            super().__init__()
            self.self_attn = nn.Linear(256, 256)
            self.mlp = nn.Sequential(nn.Linear(256, 512), nn.ReLU(), nn.Linear(512, 256))

        def forward(self, x):
            return self.mlp(self.self_attn(x))

    blk = Block()
    mgr = ActivationManager(CheckpointPolicy(checkpoint_attention=False, checkpoint_ffn=True, min_trainable_params=1000))
    assert mgr.hook_into_model(blk) == ["mlp"]
    x = torch.randn(4, 256, requires_grad=True)
    blk(x).sum().backward()
    g1 = blk.mlp[0].weight.grad.clone()
    mgr.unhook()
    blk.zero_grad()
    blk(x).sum().backward()
    assert torch.allclose(g1, blk.mlp[0].weight.grad)
    mgr.checkpoint_attention().checkpoint_ffn(False)
    assert mgr.hook_into_model(blk) == ["self_attn"]
    est = ActivationManager.estimate_memory_saving(12, 768, 512, 32)
    assert abs(est["attention_mb"] - 301.99) < 1 and abs(est["total_gb"] - 1.51) < 0.01


def test_memory_tracker_and_execution_plan():
    t = MemoryTracker(history=4)
    for _ in range(10):
        t.snapshot()
    assert len(t.snapshots) == 4 and not t.possible_leak()
    p = ExecutionPlan.from_model(_mlp(), batch_size=2, seq_len=4)
    assert p.num_forward_ops == 3 and p.estimate_memory_gb() > 0 and p.estimate_time_seconds() > 0


def test_peer_barrier_protocol_model_under_random_interleavings():
    """The flag-barrier state machine of the peer barrier kernel, run on CPU threads with randomised
    delays: nobody leaves a barrier before everyone entered it, data written before is visible after,
    the epoch comparison survives the 32-bit wrap, and a missing rank ends the others' waits with a
    time-out instead of a hang."""
    from zenyx_b200.ops import _ext

    h = _ext.host()
    for seed in range(3):
        r = h.barrier_model(4, 150, 0, seed)
        assert r["violations"] == 0 and r["timeouts"] == 0 and r["rounds_done"] == 150, r
    r = h.barrier_model(8, 80, 0xFFFFFFC0, 7)          # crosses the wrap of the 32-bit epoch
    assert r["violations"] == 0 and r["timeouts"] == 0 and r["rounds_done"] == 80, r
    r = h.barrier_model(3, 40, 0, 9, absent_rank=1, absent_from_round=10, timeout_us=20000)
    assert r["violations"] == 0 and r["timeouts"] >= 1 and r["rounds_done"] == 10, r


def test_attention_tile_iteration_equals_a_plain_scan():
    """The mask-aware tile iteration of the attention kernels (jumps over excluded runs, division-free
    cursors, the forward kernel's pair walk), compiled for the host, against a brute-force scan with the
    same mask predicate: dense, causal, one- and two-sided windows, global blocks, and position layouts
    in one, two (zigzag) and many out-of-order chunks, for every Q tile and every KV tile."""
    import random

    from zenyx_b200.ops import _ext

    h = _ext.host()
    rng = random.Random(0)
    cases = [(False, 0, 0, [0], [0], 8, 8), (True, 0, 0, [0], [0], 16, 16),
             (True, 32, 64, [0], [0], 256, 256),                              # 32K tokens, 4096 window, global every 64
             (True, 2, 4, [0, 3 * 1024], [0, 3 * 1024], 8, 8),                # zigzag rank 0 of a ring of 2
             (True, 3, 0, [1024, 2048], [0, 3 * 1024], 8, 8)]                 # Q of rank 1 against KV of rank 0
    for _ in range(60):
        nq, nk = rng.choice([1, 2, 4, 8]), rng.choice([1, 2, 4, 8])
        per_q, per_k = rng.choice([1, 2, 3, 8]), rng.choice([1, 2, 5, 8])
        span = 64
        qc = [128 * per_q * c for c in rng.sample(range(span), nq)]
        kc = [128 * per_k * c for c in rng.sample(range(span), nk)]
        cases.append((rng.random() < 0.6, rng.choice([0, 1, 2, 5, 9]), rng.choice([0, 1, 3, 4, 16]), qc, kc, per_q, per_k))
    for causal, wb, ge, qc, kc, per_q, per_k in cases:
        bad = h.tile_iter_mismatches(causal, wb, ge, qc, kc, per_q, per_k)
        assert bad == 0, (causal, wb, ge, qc, kc, per_q, per_k, bad)


def test_tracing_helpers_and_loop_metrics(tmp_path):
    """PhaseTimer accumulates per-phase time, trace ranges are no-ops without a GPU, and the training loop's
    JSON-lines records carry tokens/s, MFU, ring and data-parallel degree for the flagship."""
    import json

    from zenyx_b200.models import LlamaConfig
    from zenyx_b200.train import Trainer, TrainerConfig, loop
    from zenyx_b200.utils import tracing

    t = tracing.PhaseTimer()
    with t.phase("a"):
        with tracing.trace_range("inner"):
            sum(range(1000))
    with t.phase("a"):
        pass
    assert set(t.summary()) == {"a"} and t.summary()["a"] >= 0.0
    tracing.enable(True)
    assert tracing.enabled()
    with tracing.trace_range("x"):
        pass
    tracing.enable(False)
    cfg = LlamaConfig.tiny(n_layers=1, d_model=64, n_heads=2, n_kv_heads=1, ffn_dim=96, vocab_size=128)
    tr = Trainer(cfg, TrainerConfig(lr=1e-3, seq_len=128, global_batch=2))

    def data():
        g = torch.Generator().manual_seed(0)
        while True:
            x = torch.randint(0, 128, (2, 128), generator=g)
            yield x, x

    path = str(tmp_path / "metrics.jsonl")
    loop.run(tr, data(), cfg=loop.LoopConfig(steps=2, log_every=0, metrics_path=path, tokens_per_step=256))
    tr.close()
    recs = [json.loads(l) for l in open(path)]
    assert len(recs) == 2 and all(k in recs[0] for k in ("step", "loss", "tokens_per_s", "mfu", "ring_degree", "dp_degree"))
    assert recs[0]["mfu"] > 0
