"""Benchmark entry points (kernel microbenchmarks, ring attention, 8B training step, tiering)."""
