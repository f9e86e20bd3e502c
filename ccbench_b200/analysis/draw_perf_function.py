"""Rank x function heat map of the time spent per intercepted function, from the perf
wrapper CSVs. Counterpart of the reference's scripts/statistic/draw_perf_function.py
(:30-58 reader, heat map per rank and function). Headless: PNG only.

    python -m ccbench_b200.analysis.draw_perf_function --perf-dir perf_files --save perf.png
"""
from __future__ import annotations

import argparse
import csv
import glob
import os


def totals(perf_dir):
    table, funcs = {}, set()
    for path in sorted(glob.glob(os.path.join(perf_dir, "perf_function_*.csv")) + glob.glob(os.path.join(perf_dir, "perf_nccl_*.csv"))):
        rank = os.path.splitext(os.path.basename(path))[0].rsplit("_", 1)[-1]
        with open(path) as f:
            for row in csv.DictReader(f):
                d = row.get("device_duration") or row.get("duration") or "0"
                table.setdefault(rank, {}).setdefault(row["func_name"], [0.0, 0])
                table[rank][row["func_name"]][0] += float(d or 0)
                table[rank][row["func_name"]][1] += 1
                funcs.add(row["func_name"])
    return table, sorted(funcs)


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--perf-dir", default="perf_files")
    ap.add_argument("--save", default="perf_function.png")
    a = ap.parse_args(argv)
    table, funcs = totals(a.perf_dir)
    if not table:
        print("no perf CSVs under", a.perf_dir)
        return 1
    import numpy as np

    ranks = sorted(table, key=lambda r: int(r) if r.isdigit() else 0)
    grid = np.array([[table[r].get(f, [0.0, 0])[0] * 1e3 for f in funcs] for r in ranks])
    try:
        import matplotlib
    except ImportError:   # headless host without matplotlib: plain PNG + legend file
        from ._png import heatmap

        heatmap(a.save, grid, [f"rank {r}" for r in ranks], "functions, left to right: " + ", ".join(funcs), "total time (ms)",
                cell=(48, 24))
    else:
        matplotlib.use("Agg")
        import matplotlib.pyplot as plt

        fig, ax = plt.subplots(figsize=(max(4, len(funcs)), max(3, 0.4 * len(ranks) + 2)))
        im = ax.imshow(grid, aspect="auto", cmap="magma")
        ax.set_xticks(range(len(funcs)))
        ax.set_xticklabels(funcs, rotation=45, ha="right", fontsize=7)
        ax.set_yticks(range(len(ranks)))
        ax.set_yticklabels(ranks)
        ax.set_ylabel("rank")
        fig.colorbar(im, ax=ax, label="total time (ms)")
        fig.tight_layout()
        fig.savefig(a.save, dpi=120)
    for r in ranks:
        print(r, {f: (round(v[0] * 1e3, 3), v[1]) for f, v in table[r].items()})
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
