"""Heat map of the daemon samples (perf_files/perf_<device>_<host>.csv) against time,
one row per device, optionally restricted to the devices that perf_files/map.csv
assigns to ranks. Counterpart of the reference's scripts/statistic/draw_hardware.py
(:36-42 CSV reader, :190-213 map.csv, :256-300 heat map). Always headless: the figure
is written as PNG; an interactive window is not available on these machines.

    python -m ccbench_b200.analysis.draw_hardware --perf-dir perf_files --metric gpu_util --save hw.png
"""
from __future__ import annotations

import argparse
import csv
import glob
import os


def load_device_csv(path):
    with open(path) as f:
        rows = list(csv.DictReader(f))
    t = [float(r["timestamp_sec"]) for r in rows]
    cols = {k: [float(r[k]) if r[k] else float("nan") for r in rows] for k in (rows[0].keys() if rows else []) if k != "timestamp_sec"}
    return t, cols


def load_map(path):
    if not os.path.exists(path):
        return []
    with open(path) as f:
        return [(int(r["rank"]), r["node"], r["device_type"], int(r["device_number"])) for r in csv.DictReader(f)]


def collect(perf_dir, metric, device_class=None, t_min=None, t_max=None):
    series = {}
    for path in sorted(glob.glob(os.path.join(perf_dir, "perf_*.csv"))):
        name = os.path.basename(path)[len("perf_"):-len(".csv")]
        if name.startswith(("function_", "nccl_")) or name == "map":
            continue
        if device_class and not name.startswith(device_class):
            continue
        t, cols = load_device_csv(path)
        if metric not in cols:
            continue
        pts = [(a, b) for a, b in zip(t, cols[metric]) if (t_min is None or a >= t_min) and (t_max is None or a <= t_max)]
        if pts:
            series[name] = pts
    return series


def _grid(series, bins):
    import numpy as np

    names = sorted(series)
    t0 = min(p[0][0] for p in series.values())
    t1 = max(p[-1][0] for p in series.values())
    grid = np.full((len(names), bins), np.nan)
    for i, n in enumerate(names):
        for t, v in series[n]:
            j = min(bins - 1, int((t - t0) / max(t1 - t0, 1e-9) * bins))
            grid[i, j] = v
    return names, t0, t1, grid


def plot(series, metric, path, bins=200):
    names, t0, t1, grid = _grid(series, bins)
    try:
        import matplotlib
    except ImportError:   # headless host without matplotlib: plain PNG + legend file
        from ._png import heatmap

        heatmap(path, grid, names, f"time, {t0:.3f} s .. {t1:.3f} s in {bins} bins", metric, cell=(4, 18))
        return path
    matplotlib.use("Agg")
    import matplotlib.pyplot as plt

    fig, ax = plt.subplots(figsize=(10, max(2, 0.3 * len(names) + 1)))
    im = ax.imshow(grid, aspect="auto", extent=[t0, t1, len(names), 0], cmap="viridis")
    ax.set_yticks([i + 0.5 for i in range(len(names))])
    ax.set_yticklabels(names, fontsize=6)
    ax.set_xlabel("time (s)")
    fig.colorbar(im, ax=ax, label=metric)
    fig.tight_layout()
    fig.savefig(path, dpi=120)
    return path


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--perf-dir", default="perf_files")
    ap.add_argument("--metric", default="gpu_util")
    ap.add_argument("--device-class", default=None, help="cpu | gpu | ib | pcie")
    ap.add_argument("--t-min", type=float, default=None)
    ap.add_argument("--t-max", type=float, default=None)
    ap.add_argument("--save", default="hardware.png")
    a = ap.parse_args(argv)
    s = collect(a.perf_dir, a.metric, a.device_class, a.t_min, a.t_max)
    if not s:
        print("no samples for metric", a.metric)
        return 1
    plot(s, a.metric, a.save)
    print("wrote", a.save, "devices:", len(s), "ranks mapped:", len(load_map(os.path.join(a.perf_dir, "map.csv"))))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
