from .bandwidth import BandwidthAwareScheduler, BandwidthSample
from .belady import BeladyApproxCache
from .engine import StreamingConfig, StreamingExecutionEngine
from .kv_tiering import KVBlockRef, KVTierManager, build_ring_timeline
from .parameter_streamer import LayerWeightStreamer, ParameterStore
from .precision import dequantize_for_bf16_compute, quantize_to_fp8_storage

__all__ = ["StreamingExecutionEngine", "StreamingConfig", "LayerWeightStreamer", "ParameterStore", "KVTierManager",
           "KVBlockRef", "build_ring_timeline", "BeladyApproxCache", "BandwidthAwareScheduler", "BandwidthSample",
           "quantize_to_fp8_storage", "dequantize_for_bf16_compute"]
