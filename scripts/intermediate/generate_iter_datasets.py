#!/usr/bin/env python3
"""Dataset files of 512 MB per category from captured tensors (or synthetic ones): the
reference's script name; the work is done by ccbench_b200.datasets."""
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))
from ccbench_b200.datasets import main  # noqa: E402

if __name__ == "__main__":
    raise SystemExit(main(["--size", "512mb", *sys.argv[1:]]))
