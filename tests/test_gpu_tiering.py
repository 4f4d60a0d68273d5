"""The KV tiering manager in real mode on a GPU: blocks spill from a capped HBM budget to pinned host
memory and a file, come back through the prefetch path, and carry the right bytes."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("with_file", [False, True])
def test_manager_serves_the_planned_accesses_from_all_tiers(tmp_path, with_file):
    from zenyx_b200.train.belayd_kv_cache_tiering import BeladyKVCacheTieringManager

    ring, layers, ctx_len, bt, hkv, d = 4, 3, 4 * 8 * 256, 256, 2, 128
    block_bytes = 2 * bt * hkv * d * 2
    mgr = BeladyKVCacheTieringManager(num_devices=ring, context_length=ctx_len, num_layers=layers, num_kv_heads=hkv,
                                      head_dim=d, tier_block_tokens=bt, hbm_budget_bytes=6 * block_bytes,
                                      dram_budget_bytes=(5 * block_bytes) if with_file else None,
                                      nvme_path=str(tmp_path / "kv.bin") if with_file else None, simulate=False,
                                      rank=0, lookahead=2)
    assert mgr.total_kv_bytes() > mgr.hbm_budget_bytes
    gen = torch.Generator(device="cuda").manual_seed(0)
    truth = {}
    for layer in range(layers):
        for b in range(mgr.blocks_per_layer):
            kv = torch.randn(2, bt, hkv, d, device="cuda", generator=gen).bfloat16()
            truth[mgr.block_id(layer, b)] = kv.clone()
            mgr.register(layer, b, kv)
    plan = mgr.plan()
    for _ in range(2):
        mgr.step_begin()
        for bid in plan.ids:
            layer, b = divmod(bid, mgr.blocks_per_layer)
            got = mgr.acquire(layer, b)
            torch.cuda.current_stream().synchronize()
            assert torch.equal(got.view(2, bt, hkv, d), truth[bid]), bid
            assert len(mgr._hbm) * block_bytes <= mgr.hbm_budget_bytes
        mgr.step_end()
    st = mgr.stats()
    assert st.accesses == 2 * len(plan.ids) and st.misses > 0 and st.bytes_h2d > 0
    assert st.peak_hbm_bytes <= mgr.hbm_budget_bytes
    if with_file:
        assert st.bytes_nvme_write > 0 and st.bytes_nvme_read > 0
    mgr.close()


def test_ring_attention_over_tiered_kv_single_rank(capsys):
    """The tiered ring benchmark at ring degree 1 on a small case: every layer's K/V goes through the manager
    under a budget smaller than one layer, the attention kernels run on what it hands out, the step reports
    spills and a finite time."""
    import json

    from zenyx_b200.bench import ring_tiering

    ring_tiering.main(["--seq-len", "8192", "--layers", "3", "--block-tokens", "1024", "--hbm-gb", "0.004",
                       "--steps", "2"])
    rec = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert rec["ring_degree"] == 1 and rec["layers"] == 3 and rec["value"] > 0
    assert rec["share_kv_bytes"] > rec["hbm_budget_bytes"]
    assert rec["measured"]["misses"] > 0 and rec["measured"]["bytes_h2d"] > 0
    assert rec["measured"]["peak_hbm_bytes"] <= rec["hbm_budget_bytes"]
