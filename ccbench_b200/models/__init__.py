"""Synthetic workloads: the data distributions and shapes the benchmarks run on."""
