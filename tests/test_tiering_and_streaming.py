import itertools
import os

import numpy as np
import pytest
import torch
import torch.nn as nn

from zenyx_b200.ops import _ext
from zenyx_b200.streaming import (BandwidthAwareScheduler, BandwidthSample, BeladyApproxCache, KVTierManager,
                                  LayerWeightStreamer, ParameterStore, StreamingExecutionEngine, build_ring_timeline,
                                  dequantize_for_bf16_compute, quantize_to_fp8_storage)
from zenyx_b200.train.belayd_kv_cache_tiering import BeladyKVCacheTieringManager, RingAttentionAccessSequence


def test_belady_cache_prefers_farthest_next_use():
    cache = BeladyApproxCache(capacity=2)
    cache.update_future("a", 1)
    cache.update_future("b", 100)
    cache.update_future("c", 2)
    cache.touch("a")
    cache.touch("b")
    assert cache.touch("c") == ["b"]
    by = BeladyApproxCache(capacity=100, unit="bytes")
    by.update_future("x", 5)
    by.update_future("y", 9)
    by.touch("x", 60)
    assert by.touch("y", 60) == ["x"]


def test_bandwidth_scheduler():
    s = BandwidthAwareScheduler(1.0)
    assert s.should_throttle(BandwidthSample(2.0, 1.0)) and not s.should_throttle(BandwidthSample(0.5, 1.0))
    assert s.should_throttle(BandwidthSample(1.0, 0.0))
    assert s.throttle_ms(BandwidthSample(3.0, 1.0)) == 2.0


def test_fp8_storage_roundtrip_is_real_e4m3():
    x = torch.randn(64, 64)
    q, scale = quantize_to_fp8_storage(x)
    assert q.dtype == torch.float8_e4m3fn
    y = dequantize_for_bf16_compute(q, scale)
    assert y.shape == x.shape and y.dtype == torch.bfloat16
    assert ((y.float() - x).norm() / x.norm()).item() < 0.06


def _brute_force_min_misses(ids, cap_blocks):
    """Optimal number of misses for unit-size blocks by exhaustive search (tiny traces only)."""
    best = [len(ids) + 1]

    def rec(i, resident, misses):
        if misses >= best[0]:
            return
        if i == len(ids):
            best[0] = misses
            return
        b = ids[i]
        if b in resident:
            rec(i + 1, resident, misses)
            return
        if len(resident) < cap_blocks:
            rec(i + 1, resident | {b}, misses + 1)
            return
        for victim in resident:
            rec(i + 1, (resident - {victim}) | {b}, misses + 1)
        rec(i + 1, resident, misses + 1)  # bypass

    rec(0, frozenset(), 0)
    return best[0]


def test_belady_min_is_optimal_on_small_traces():
    host = _ext.host()
    rng = np.random.default_rng(0)
    for _ in range(30):
        n_blocks, cap = int(rng.integers(3, 6)), int(rng.integers(1, 4))
        ids = [int(x) for x in rng.integers(0, n_blocks, size=9)]
        res = host.belady_min(ids, [10] * n_blocks, cap * 10)
        assert res["misses"] == _brute_force_min_misses(ids, cap), (ids, cap)
        lru = host.lru_trace(ids, [10] * n_blocks, cap * 10)
        assert res["misses"] <= lru["misses"]
        assert res["peak_resident_bytes"] <= cap * 10
        assert res["hits"] + res["misses"] == len(ids)


def test_belady_min_respects_bytes():
    host = _ext.host()
    res = host.belady_min([0, 1, 2, 0, 1, 2], [30, 30, 50], 60)
    assert res["peak_resident_bytes"] <= 60 and res["hits"] >= 1


def test_access_sequence_shape_and_order():
    seq = RingAttentionAccessSequence(num_devices=4, num_layers=2, blocks_per_device=3)
    acc = seq.accesses()
    assert len(acc) == 2 * 2 * 4 * 4 * 3           # phases x layers x steps x readers x blocks
    assert [a.t for a in acc] == sorted(a.t for a in acc)
    fwd = [a for a in acc if a.phase == "forward"]
    assert fwd[0].layer == 0 and fwd[-1].layer == 1
    bwd = [a for a in acc if a.phase == "backward"]
    assert bwd[0].layer == 1 and bwd[-1].layer == 0
    # at ring step s device r reads the owner (r - s) mod R
    for a in acc:
        step = a.t % 4
        assert a.owner == (a.reader - step) % 4
    local = seq.for_device(2)
    assert all(a.owner == 2 for a in local) and len(local) == len(acc) // 4
    assert seq.next_use(2, 0, 0, 0) is not None
    assert build_ring_timeline(3) == {"forward": [0, 1, 2], "backward": [2, 1, 0]}


def test_sparse_pattern_drops_ring_steps():
    from zenyx_b200.train.sparse_ring_attention import SparsePattern

    dense = RingAttentionAccessSequence(8, 1, 1, seq_len=262144)
    sparse = RingAttentionAccessSequence(8, 1, 1, seq_len=262144,
                                         sparse_pattern=SparsePattern(window_tokens=4096, global_every=0))
    assert len(sparse) < len(dense)


def test_manager_plan_and_simulation():
    m = BeladyKVCacheTieringManager(num_devices=8, context_length=4096, num_layers=12)
    assert m.simulate_mode
    p = m.plan()
    assert p.misses == 12 and p.hit_rate > 0.9          # everything fits: only cold misses
    tight = BeladyKVCacheTieringManager(num_devices=8, context_length=1 << 20, num_layers=8, hbm_budget_bytes=1 << 30,
                                        tier_block_tokens=16384, dram_budget_bytes=2 << 30)
    assert tight.total_kv_bytes() > tight.hbm_budget_bytes
    plan = tight.plan()
    assert plan.peak_resident_bytes <= tight.hbm_budget_bytes
    assert plan.misses <= tight.lru_baseline()["misses"]
    fast = tight.simulate({"pcie_gbs": 50.0, "nvme_gbs": 6.0}, compute_ms_per_access=5.0)
    slow = tight.simulate({"pcie_gbs": 1.0, "nvme_gbs": 0.5}, compute_ms_per_access=5.0)
    assert slow.exposed_stall_ms > fast.exposed_stall_ms
    assert fast.bytes_h2d == plan.misses * tight.block_bytes and fast.bytes_nvme_read > 0


def test_file_tier_roundtrip(tmp_path):
    host = _ext.host()
    tier = host.FileTier(str(tmp_path / "kv.bin"), 8192, 4, 2, True)
    a = torch.arange(2048, dtype=torch.float32)
    b = torch.zeros(2048, dtype=torch.float32)
    # page-aligned buffers for O_DIRECT; fall back silently when the file system refuses it
    buf = torch.empty(8192 + 4096, dtype=torch.uint8)
    off = (-buf.data_ptr()) % 4096
    src = buf[off: off + 8192].view(torch.float32)
    src.copy_(a)
    assert tier.wait(tier.write_async(3, src.data_ptr(), 8192)) == 0
    src.zero_()
    assert tier.wait(tier.read_async(3, src.data_ptr(), 8192)) == 0
    b.copy_(src)
    assert torch.equal(a, b) and tier.bytes_written == 8192 and tier.bytes_read == 8192
    with pytest.raises(RuntimeError):
        tier.write_async(9, src.data_ptr(), 8192)


def test_kv_tier_manager_tiers_and_file(tmp_path):
    kv = KVTierManager(t0_capacity=1, t1_capacity=1, device=torch.device("cpu"), nvme_path=str(tmp_path / "t2.bin"),
                       block_bytes=4096, t2_slots=8)
    blocks = {i: torch.randn(32, 32) for i in range(3)}
    for i, t in blocks.items():
        kv.put(i, t)
    assert all(kv.location(i) == "t2" for i in blocks)
    for i in (0, 1, 2, 0):
        got = kv.prefetch_to_t0(i)
        assert torch.equal(got, blocks[i])
        assert len(kv.t0) <= 1 and len(kv.t1) <= 1


def test_streamer_binds_weights_and_engine_runs():
    torch.manual_seed(0)
    model = nn.Sequential(nn.Linear(8, 16), nn.ReLU(), nn.Linear(16, 4))
    store = ParameterStore()
    store.register("0", model[0])
    st = LayerWeightStreamer(store, "cpu")
    ref = model[0].weight.detach().clone()
    with torch.no_grad():
        model[0].weight.zero_()
    st.bind("0", model[0])
    assert torch.equal(model[0].weight, ref)
    eng = StreamingExecutionEngine(model, device=torch.device("cpu"))
    eng.kv_manager.put("b0", torch.randn(4))
    loss = eng.run_forward_backward(torch.randn(2, 8), torch.randn(2, 4), nn.MSELoss())
    assert loss >= 0 and model[0].weight.grad is not None and len(eng.last_samples) == 3


def test_tiered_ring_benchmark_follows_the_managers_plan():
    """The acquires that bench/ring_tiering.py makes per step are exactly the manager's planned accesses of the
    rank, in order, for every rank of a ring: the manager then evicts and prefetches by its Belady plan instead of
    falling back to out-of-plan handling."""
    from zenyx_b200.bench.ring_tiering import acquire_order
    from zenyx_b200.train.belayd_kv_cache_tiering import BeladyKVCacheTieringManager

    for ring, layers, nb in ((1, 3, 4), (2, 4, 8), (4, 2, 4), (8, 3, 2)):
        bt = 256
        for rank in range(ring):
            mgr = BeladyKVCacheTieringManager(num_devices=ring, context_length=ring * nb * bt, num_layers=layers,
                                              num_kv_heads=2, head_dim=64, tier_block_tokens=bt,
                                              hbm_budget_bytes=3 * 2 * bt * 2 * 64 * 2, simulate=True, rank=rank)
            assert mgr.blocks_per_layer == nb
            ids = [layer * nb + b for layer, b in acquire_order(ring, layers, nb)]
            assert ids == list(mgr.plan().ids), (ring, layers, nb, rank)
