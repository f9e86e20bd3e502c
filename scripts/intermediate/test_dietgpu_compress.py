#!/usr/bin/env python3
"""Ratio and throughput of the lossless GPU codec on one dataset file: the reference's
script name; the work is done by ccbench_b200.bench.lossless_ratio."""
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))
from ccbench_b200.bench.lossless_ratio import main  # noqa: E402

if __name__ == "__main__":
    raise SystemExit(main(sys.argv[1:] or ["dataset/kv/kv_cache_512mb.f32", "--sizes", "256M"]))
