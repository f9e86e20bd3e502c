"""CPU-only benchmark: 2 (or N) MPI ranks, ring MPI_Allreduce(SUM) of a 1 Mi-element
float32 buffer per rank, values N(0,1) seeded 0 + rank, every hop quantised to int8 in
blocks of 128 with an absmax/127 scale (the MPI interposer + the int8 codec wrapper
under the unmodified allreduce driver). Reports latency, compression ratio and
max-abs / RMSE / relative-L2 deviation against the uncompressed float64 sum.

    python -m ccbench_b200.bench.config1_cpu [--ranks 2] [--elements 1048576] [--iters 10]

Uses the installed MPI when mpicc/mpirun exist, else the bundled single-host subset."""
from __future__ import annotations

import argparse
import json
import os
import re
import shutil
import tempfile
from pathlib import Path

import numpy as np

from .. import launch as launcher
from ..native_build import BIN, ROOT, build_c_targets


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--ranks", type=int, default=2)
    ap.add_argument("--elements", type=int, default=1 << 20)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--block", type=int, default=128)
    a = ap.parse_args(argv)
    build_c_targets()
    work = Path(tempfile.mkdtemp(prefix="ccb_config1_"))
    data = work / "data"
    data.mkdir()
    xs = []
    for r in range(a.ranks):
        x = np.random.default_rng(0 + r).standard_normal(a.elements).astype(np.float32)
        x.tofile(data / f"rank_{r}.bin")
        xs.append(x)
    exact = np.sum(np.stack(xs).astype(np.float64), axis=0)
    nbytes = a.elements * 4
    libs = BIN / "libs"
    out = {}
    for label, preload in (("uncompressed", ""), ("int8_block", f"{libs / 'libperfmpi.so'}:{libs / 'libmpi_int8.so'}:{libs / 'libplain_mpi_compress.so'}")):
        run = work / label
        run.mkdir()
        env = {"CCB_MINIMPI_JOB": f"c1{os.getpid()}{label[:2]}", "BENCH_DIR": str(ROOT), "DS_TYPE": "folder", "DS_SUFFIX": ".bin",
               "MPI_INT8_BLOCK": str(a.block), "PERF_OUTPUT_DIR": str(run / "perf_files"), "PYTHONPATH": str(ROOT)}
        cmd = [str(BIN / "mpi/allreduce/allreduce"), "-L", str(nbytes), "-i", str(a.iters), "-w", "3", "-d", "float", "-f", str(data),
               "-b", "-B", str(run / "AllReduce")]
        rcs, outs = launcher.launch(a.ranks, cmd, preload, env, cwd=str(run), timeout=600, capture=True)
        if any(rcs):
            print(outs[0])
            return 1
        m = re.search(r"User: avg=\s*([\d.]+) us, min=\s*([\d.]+) us, max=\s*([\d.]+) us", outs[0])
        got = np.fromfile(run / "AllReduce_user.bin", dtype=np.float32).astype(np.float64)
        d = got - exact
        res = {"latency_us_max_over_ranks": float(m.group(3)) if m else None, "max_abs_err": float(np.abs(d).max()),
               "rmse": float(np.sqrt(np.mean(d * d))), "rel_l2": float(np.linalg.norm(d) / np.linalg.norm(exact))}
        if preload:
            ratios = []
            for f in (run / "perf_files").glob("perf_function_*.csv"):
                for line in f.read_text().splitlines()[1:]:
                    p = line.split(",")
                    if p[0] == "mpi_compress" and len(p) > 6 and p[6]:
                        ratios.append(float(p[6]))
            res["compression_ratio"] = float(np.mean(ratios)) if ratios else None
        out[label] = res
    print(json.dumps({"config": {"ranks": a.ranks, "elements": a.elements, "dtype": "float32", "block": a.block,
                                 "algorithm": "ring reduce-scatter + all-gather, codec round trip per hop",
                                 "mpi": "system" if shutil.which("mpirun") else "bundled single-host subset"}, **out}, indent=2))
    shutil.rmtree(work, ignore_errors=True)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
