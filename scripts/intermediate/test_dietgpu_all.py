#!/usr/bin/env python3
"""Ratio of the lossless GPU codec on every dataset category at sizes from 8 KB to 512 MB:
the reference's script name; the work is done by ccbench_b200.bench.lossless_ratio."""
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))
from ccbench_b200.bench.lossless_ratio import main  # noqa: E402

if __name__ == "__main__":
    raise SystemExit(main(sys.argv[1:] or ["dataset"]))
