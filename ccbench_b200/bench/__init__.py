"""Benchmarks: size sweep, configurations 1-5, phase timelines, profiler cases, report tables."""
