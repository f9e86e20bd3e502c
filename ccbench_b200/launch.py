"""Minimal local launcher: start N ranks of a benchmark binary on this host with the
rank environment the NCCL bridge reads (OMPI_COMM_WORLD_RANK / _SIZE / _LOCAL_RANK),
one GPU per rank, and wait for all of them. It stands in for `mpirun -np N` on hosts
without MPI (the reference's NCCL benchmarks only take the rank from the launcher's
environment: run_codes/benchmark-core/src/nccl/nccl_utils.c:47-68).

    python -m ccbench_b200.launch -n 4 [--preload a.so:b.so] [--env K=V ...] -- bin/nccl/allreduce/allreduce -m 1024:1048576:4
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
import time


def clean_runtime_dirs(cwd: str) -> None:
    """What the generated run script does before each phase: stale rendezvous and
    aggregation files of an earlier run must not be picked up."""
    for d in ("nccl_id_file", os.path.join("runtime_files", "nccl_agg")):
        p = os.path.join(cwd, d)
        shutil.rmtree(p, ignore_errors=True)
        os.makedirs(p, exist_ok=True)


def launch(n: int, cmd: list[str], preload: str = "", env: dict | None = None, cwd: str | None = None,
           timeout: float | None = None, capture: bool = False):
    cwd = cwd or os.getcwd()
    clean_runtime_dirs(cwd)
    procs = []
    for r in range(n):
        e = dict(os.environ)
        e.update({"OMPI_COMM_WORLD_RANK": str(r), "OMPI_COMM_WORLD_SIZE": str(n), "OMPI_COMM_WORLD_LOCAL_RANK": str(r)})
        if env:
            e.update(env)
        if preload:
            e["LD_PRELOAD"] = preload + (":" + e["LD_PRELOAD"] if e.get("LD_PRELOAD") else "")
        out = subprocess.PIPE if capture else (None if r == 0 else subprocess.DEVNULL)
        procs.append(subprocess.Popen(cmd, cwd=cwd, env=e, stdout=out, stderr=subprocess.STDOUT if capture else None, text=capture))
    deadline = time.time() + timeout if timeout else None
    outs, rcs = [], []
    for p in procs:
        try:
            o, _ = p.communicate(timeout=max(1.0, deadline - time.time()) if deadline else None)
        except subprocess.TimeoutExpired:
            for q in procs:
                if q.poll() is None:
                    q.kill()
            o, _ = p.communicate()
        outs.append(o)
        rcs.append(p.returncode)
    return rcs, outs


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("-n", type=int, required=True)
    ap.add_argument("--preload", default="")
    ap.add_argument("--env", action="append", default=[])
    ap.add_argument("--timeout", type=float, default=None)
    ap.add_argument("cmd", nargs=argparse.REMAINDER)
    a = ap.parse_args(argv)
    cmd = a.cmd[1:] if a.cmd and a.cmd[0] == "--" else a.cmd
    env = dict(kv.split("=", 1) for kv in a.env)
    rcs, _ = launch(a.n, cmd, a.preload, env, timeout=a.timeout)
    return max(abs(rc) for rc in rcs)


if __name__ == "__main__":
    sys.exit(main())
