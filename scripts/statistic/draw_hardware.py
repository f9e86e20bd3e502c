#!/usr/bin/env python3
"""The reference's script name; the work is done by ccbench_b200.analysis.draw_hardware (plots go to PNG
files, no window)."""
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))
from ccbench_b200.analysis.draw_hardware import main  # noqa: E402

if __name__ == "__main__":
    raise SystemExit(main(sys.argv[1:]))
