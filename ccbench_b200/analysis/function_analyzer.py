"""Timeline analysis of the perf-wrapper CSVs (perf_files/perf_function_<rank>.csv,
perf_nccl_<rank>.csv): classify every row as communication or compression by its
function name, estimate the true duration of asynchronous calls whose recorded
duration is only the enqueue time, and sweep the merged timeline into
communication / compression / overlap / idle time per rank.

Input and rules follow the reference's scripts/statistic/function_analyzer.py: rows
carry timestamp_us (microseconds) and duration (SECONDS) (:175-273); a call shorter
than 10 us is treated as asynchronous and its duration is interpolated from
results/pingpong.csv by message size and intra/inter node (:97-148, 241-254); the
sweep is :280-355. Here a `device_duration` column, when present (perfnccl with
PERF_NCCL_DEVICE_TIME=1), is preferred over the estimate.

    python -m ccbench_b200.analysis.function_analyzer --perf-dir perf_files [--pingpong results/pingpong.csv] [--save out.png]
"""
from __future__ import annotations

import argparse
import bisect
import csv
import glob
import json
import os

COMM = ("send", "recv", "allreduce", "all_reduce", "bcast", "broadcast", "allgather", "reducescatter", "reduce_scatter",
        "alltoall", "gather", "scatter", "reduce", "sendrecv", "exchange")
COMP = ("compress", "decompress", "decompreducecomp", "decompressreduce", "quant", "homomorphic", "codec")
ASYNC_THRESHOLD_US = 10.0


def classify(func: str) -> str:
    f = func.lower()
    if any(k in f for k in COMP):
        return "comp"
    if any(k in f for k in COMM):
        return "comm"
    return "other"


def load_pingpong(path):
    """-> {(kind, 'intra'|'inter'): sorted [(msg_size, time_us)]}, kind in send/recv."""
    table = {}
    if not path or not os.path.exists(path):
        return table
    with open(path) as f:
        for row in csv.DictReader(f):
            try:
                size = float(row["msg_size"])
            except (KeyError, ValueError):
                continue
            where = row.get("comm_type", "intra") or "intra"
            for kind, col in (("send", "send0_us"), ("recv", "recv0_us")):
                if row.get(col):
                    table.setdefault((kind, where), []).append((size, float(row[col])))
    for v in table.values():
        v.sort()
    return table


def interpolate(points, size):
    if not points:
        return None
    xs = [p[0] for p in points]
    i = bisect.bisect_left(xs, size)
    if i == 0:
        return points[0][1]
    if i >= len(points):
        x0, y0 = points[-1]
        return y0 * size / x0 if x0 > 0 else y0  # bandwidth-bound extrapolation
    (x0, y0), (x1, y1) = points[i - 1], points[i]
    return y0 + (y1 - y0) * (size - x0) / (x1 - x0) if x1 > x0 else y0


def load_rank(path, pingpong):
    events = []
    with open(path) as f:
        for row in csv.DictReader(f):
            func = row.get("func_name", "")
            try:
                t0 = float(row["timestamp_us"])
            except (KeyError, ValueError):
                continue
            dur_us = float(row["duration"]) * 1e6 if row.get("duration") else 0.0
            if row.get("device_duration"):
                dur_us = max(dur_us, float(row["device_duration"]) * 1e6)
            elif dur_us <= ASYNC_THRESHOLD_US and classify(func) == "comm":
                size = float(row.get("msg_bytes") or row.get("data_bytes") or 0)
                where = "intra" if (row.get("intra", "1") or "1") not in ("0", "0.000000") else "inter"
                kind = "recv" if "recv" in func.lower() else "send"
                est = interpolate(pingpong.get((kind, where)) or pingpong.get((kind, "intra")), size)
                if est is not None:
                    dur_us = est
            events.append((t0, t0 + dur_us, classify(func), func))
    return events


def sweep(events):
    """-> dict of comm, comp, overlap, idle, span (microseconds)."""
    pts = []
    for s, e, kind, _ in events:
        if kind in ("comm", "comp") and e > s:
            pts.append((s, 0, kind))
            pts.append((e, 1, kind))
    pts.sort(key=lambda p: (p[0], -p[1]))
    active = {"comm": 0, "comp": 0}
    out = {"comm": 0.0, "comp": 0.0, "overlap": 0.0, "idle": 0.0}
    last = None
    for t, closing, kind in pts:
        if last is not None and t > last:
            dt = t - last
            if active["comm"] and active["comp"]:
                out["overlap"] += dt
            elif active["comm"]:
                out["comm"] += dt
            elif active["comp"]:
                out["comp"] += dt
            else:
                out["idle"] += dt
        active[kind] += -1 if closing else 1
        last = t
    out["span"] = (pts[-1][0] - pts[0][0]) if pts else 0.0
    return out


def analyze(perf_dir, pingpong_csv=None):
    pp = load_pingpong(pingpong_csv)
    result = {}
    for path in sorted(glob.glob(os.path.join(perf_dir, "perf_function_*.csv")) + glob.glob(os.path.join(perf_dir, "perf_nccl_*.csv"))):
        rank = os.path.splitext(os.path.basename(path))[0].rsplit("_", 1)[-1]
        ev = load_rank(path, pp)
        result[rank] = {"events": len(ev), **sweep(ev)}
    return result


def plot(result, path):
    try:
        import matplotlib
    except ImportError:
        print("matplotlib is not installed: no PNG written")
        return None
    matplotlib.use("Agg")
    import matplotlib.pyplot as plt

    ranks = sorted(result, key=lambda r: int(r) if r.isdigit() else 0)
    fig, ax = plt.subplots(figsize=(max(4, len(ranks)), 4))
    bottom = [0.0] * len(ranks)
    for key, color in (("comm", "tab:blue"), ("comp", "tab:orange"), ("overlap", "tab:green"), ("idle", "lightgray")):
        vals = [result[r][key] / 1e3 for r in ranks]
        ax.bar(ranks, vals, bottom=bottom, label=key, color=color)
        bottom = [b + v for b, v in zip(bottom, vals)]
    ax.set_xlabel("rank")
    ax.set_ylabel("time (ms)")
    ax.legend()
    fig.tight_layout()
    fig.savefig(path, dpi=120)


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--perf-dir", default="perf_files")
    ap.add_argument("--pingpong", default="results/pingpong.csv")
    ap.add_argument("--save", default="")
    a = ap.parse_args(argv)
    res = analyze(a.perf_dir, a.pingpong)
    print(json.dumps(res, indent=2))
    if a.save:
        plot(res, a.save)


if __name__ == "__main__":
    main()
