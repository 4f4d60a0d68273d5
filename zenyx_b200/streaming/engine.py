"""Layer-streaming execution of a sequential model (reference: zenyx/streaming/engine.py:18-103):
prefetch the next layer's weights, run the current layer, evict by farthest next use, throttle when
fetching outruns compute. Fetch and compute times are measured with CUDA events on a GPU (the
reference wraps asynchronous launches in wall-clock timers) and the streamed weights are bound to
the layer before it runs. KV blocks put into ``kv_manager`` are walked in ring order in backward."""
from __future__ import annotations

import time
from dataclasses import dataclass
from typing import Callable, List, Tuple

import torch
import torch.nn as nn

from .bandwidth import BandwidthAwareScheduler, BandwidthSample
from .belady import BeladyApproxCache
from .kv_tiering import KVTierManager, build_ring_timeline
from .parameter_streamer import LayerWeightStreamer, ParameterStore


@dataclass
class StreamingConfig:
    max_hbm_layers: int = 2
    kv_t0_blocks: int = 2
    kv_t1_blocks: int = 64
    bind_weights: bool = True


class StreamingExecutionEngine:
    def __init__(self, model: nn.Module, device: torch.device = torch.device("cpu"), config: StreamingConfig = None):
        self.model, self.device = model.to(device), torch.device(device)
        self.config = config or StreamingConfig()
        self.layers: List[Tuple[str, nn.Module]] = list(model.named_children()) or [("model", model)]
        self.store = ParameterStore()
        for name, layer in self.layers:
            self.store.register(name, layer)
        self.weight_streamer = LayerWeightStreamer(self.store, self.device, max_resident_layers=self.config.max_hbm_layers)
        self.cache = BeladyApproxCache(capacity=self.config.max_hbm_layers)
        self.bandwidth = BandwidthAwareScheduler()
        self.kv_manager = KVTierManager(self.config.kv_t0_blocks, self.config.kv_t1_blocks, self.device)
        self.last_samples: List[BandwidthSample] = []

    def _timed(self, fn: Callable):
        if self.device.type == "cuda":
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            out = fn()
            e.record()
            e.synchronize()
            return out, s.elapsed_time(e)
        t0 = time.perf_counter()
        out = fn()
        return out, (time.perf_counter() - t0) * 1e3

    def run_forward_backward(self, x: torch.Tensor, target: torch.Tensor, loss_fn: Callable) -> float:
        act = x.to(self.device)
        n = len(self.layers)
        self.last_samples = []
        for i, (name, layer) in enumerate(self.layers):
            if i + 1 < n:
                self.weight_streamer.prefetch(self.layers[i + 1][0])
            has_weights = self.store.get(name).numel() > 0

            def fetch():
                if has_weights and self.config.bind_weights:
                    self.weight_streamer.bind(name, layer)
                elif has_weights:
                    self.weight_streamer.get(name)

            _, fetch_ms = self._timed(fetch)
            act, compute_ms = self._timed(lambda: layer(act))
            sample = BandwidthSample(fetch_ms, compute_ms)
            self.last_samples.append(sample)
            wait = self.bandwidth.throttle_ms(sample)
            if self.bandwidth.should_throttle(sample) and wait > 0:
                time.sleep(min(wait, 50.0) / 1e3)
            # next use of this layer's weights is in backward, in reverse order
            self.cache.update_future(name, 2 * n - i)
            for victim in self.cache.touch(name):
                self.weight_streamer.evict(victim)
        loss = loss_fn(act, target.to(self.device))
        loss.backward()
        blocks = sorted(self.kv_manager.t2.keys() | self.kv_manager.t1.keys(), key=str)
        order = build_ring_timeline(len(blocks))["backward"]
        for idx in order:
            self.kv_manager.prefetch_to_t0(blocks[idx])
            self.kv_manager.evict_from_t0(blocks[idx])
        return float(loss.detach())
