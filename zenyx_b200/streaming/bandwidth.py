"""Fetch-versus-compute throttle (reference: zenyx/streaming/bandwidth.py:8-29)."""
from __future__ import annotations

from dataclasses import dataclass


@dataclass
class BandwidthSample:
    fetch_time_ms: float
    compute_time_ms: float


class BandwidthAwareScheduler:
    def __init__(self, max_fetch_to_compute_ratio: float = 1.0):
        self.max_ratio = max_fetch_to_compute_ratio

    def should_throttle(self, sample: BandwidthSample) -> bool:
        if sample.compute_time_ms <= 0:
            return True
        return sample.fetch_time_ms / sample.compute_time_ms > self.max_ratio

    def throttle_ms(self, sample: BandwidthSample) -> float:
        return max(0.0, sample.fetch_time_ms - sample.compute_time_ms * self.max_ratio)
