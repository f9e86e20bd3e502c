"""Turns result CSVs of the sweep (and of the benchmark drivers) into Markdown tables:
one row per message size, one column per (algorithm, codec), time in us and bus bandwidth,
plus the speed-up of the best compressed column over the NCCL column when there is one.

    python -m ccbench_b200.bench.report results/sweep_bf16.csv [--value busbw|time_us|algbw]
"""
from __future__ import annotations

import argparse
import csv
from collections import OrderedDict


def human(nbytes: int) -> str:
    for unit, name in ((1 << 30, "GiB"), (1 << 20, "MiB"), (1 << 10, "KiB")):
        if nbytes >= unit and nbytes % unit == 0:
            return f"{nbytes // unit} {name}"
    return f"{nbytes} B"


def load(path: str):
    """{(nranks, dtype): {size: {column: row}}} with columns in first-seen order."""
    groups: dict = OrderedDict()
    with open(path, newline="") as f:
        for row in csv.DictReader(f):
            if not row.get("msg_size", "").isdigit():
                continue   # a repeated header of an appended run
            col = f"{row['codec']} {row['algo']}" if "codec" in row else row.get("test", "time")
            g = groups.setdefault((row.get("nranks", "?"), row.get("dtype", "?")), OrderedDict())
            g.setdefault(int(row["msg_size"]), OrderedDict())[col] = row
    return groups


def table(sizes: dict, value: str = "time_us") -> str:
    cols: list[str] = []
    for by_col in sizes.values():
        cols += [c for c in by_col if c not in cols]
    key = value if any(value in r for r in next(iter(sizes.values())).values()) else "time_us_avg"
    lines = ["| bytes / rank | " + " | ".join(cols) + " | best compressed / NCCL |", "|---|" + "---|" * (len(cols) + 1)]
    for size in sorted(sizes):
        by_col = sizes[size]
        cells, times = [], {}
        for c in cols:
            r = by_col.get(c)
            cells.append("–" if r is None else f"{float(r[key]):.1f}")
            if r is not None:
                times[c] = float(r.get("time_us") or r.get("time_us_avg") or 0.0)
        nccl = next((t for c, t in times.items() if c.endswith(" nccl")), None)
        packed = [t for c, t in times.items() if not c.startswith("none ") and t > 0]
        speed = f"{nccl / min(packed):.2f} x" if nccl and packed else "–"
        lines.append(f"| {human(size)} | " + " | ".join(cells) + f" | {speed} |")
    return "\n".join(lines)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("csv")
    ap.add_argument("--value", default="time_us", choices=["time_us", "busbw", "algbw", "ref_bw", "rel_l2"])
    a = ap.parse_args(argv)
    for (n, dt), sizes in load(a.csv).items():
        print(f"### {n} ranks, {dt}, {a.value}\n")
        print(table(sizes, a.value) + "\n")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
