"""Benchmarks: collective sweeps, codec throughput, rooflines."""
