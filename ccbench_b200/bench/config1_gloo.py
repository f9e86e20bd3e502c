"""Configuration 1 without MPI: 2 (or more) CPU ranks over torch.distributed gloo, ring
AllReduce SUM of a 1 Mi-element fp32 buffer per rank (values N(0,1), seed 0 + rank), int8
blocks of 128 with an absmax/127 scale re-quantised at every hop. Prints latency,
compression ratio and max-abs / RMSE deviation against the uncompressed float64 sum.

    python -m ccbench_b200.bench.config1_gloo [--ranks 2] [--elements 1048576] [--codec int8]
"""
from __future__ import annotations

import argparse
import json
import os
import time

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from ..parallel.cpu_ring import ring_all_reduce


def _worker(rank: int, world: int, port: int, elements: int, codec: str, iters: int, q) -> None:
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.set_num_threads(max(1, (os.cpu_count() or 2) // world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    x = torch.randn(elements, generator=torch.Generator().manual_seed(rank))
    exact = x.double().clone()
    dist.all_reduce(exact)
    rows = {}
    for name in ("none", codec):
        stats: dict = {}
        ring_all_reduce(x, name)                      # warm-up
        ts = []
        for _ in range(iters):
            dist.barrier()
            t0 = time.perf_counter()
            y = ring_all_reduce(x, name, stats=stats)
            ts.append(time.perf_counter() - t0)
        t = torch.tensor([sorted(ts)[len(ts) // 2]], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        d = y.double() - exact
        rows[name] = {"latency_us_max_over_ranks": round(t.item() * 1e6, 1), "max_abs_err": d.abs().max().item(),
                      "rmse": d.pow(2).mean().sqrt().item(), "rel_l2": (d.norm() / exact.norm()).item(),
                      "compression_ratio": round(stats["raw_bytes"] / stats["wire_bytes"], 4)}
    if rank == 0:
        q.put(rows)
    dist.barrier()
    dist.destroy_process_group()


def run(ranks: int = 2, elements: int = 1 << 20, codec: str = "int8", iters: int = 5, port: int = 0) -> dict:
    import socket

    if not port:
        with socket.socket() as s:
            s.bind(("127.0.0.1", 0))
            port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, ranks, port, elements, codec, iters, q)) for r in range(ranks)]
    for p in procs:
        p.start()
    rows = q.get(timeout=600)
    for p in procs:
        p.join(timeout=120)
    return {"config": {"ranks": ranks, "elements": elements, "dtype": "float32", "block": 128, "backend": "torch.distributed gloo",
                       "algorithm": "ring reduce-scatter + all-gather, codec round trip per hop"},
            "uncompressed": rows["none"], f"{codec}_block": rows[codec]}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--ranks", type=int, default=2)
    ap.add_argument("--elements", type=int, default=1 << 20)
    ap.add_argument("--codec", default="int8", choices=["int8", "fp8"])
    ap.add_argument("--iters", type=int, default=5)
    a = ap.parse_args(argv)
    print(json.dumps(run(a.ranks, a.elements, a.codec, a.iters), indent=2))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
