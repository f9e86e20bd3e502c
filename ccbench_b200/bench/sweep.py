"""Message-size / algorithm / codec sweep of AllReduce on 1..8 GPUs, with NCCL
(torch.distributed) timed the same way as the uncompressed baseline.

    python -m torch.distributed.run --nproc-per-node N -m ccbench_b200.bench.sweep \
        --min-bytes 8 --max-bytes 1073741824 --dtype bf16 --variants none:auto,int8:twoshot,nccl

Every number is CUDA-event time on the device, maximum over ranks, after warm-up.
Columns follow the result CSV layout of this repository
(msg_size,nranks,dtype,algo,codec,time_us,algbw,busbw,ref_bw,ratio,rel_l2); `ref_bw`
is the reference's own definition 2*bytes/t
(run_codes/benchmarks/nccl/allreduce/allreduce.c:139-146).
"""
from __future__ import annotations

import argparse
import os

import torch
import torch.distributed as dist

from .. import Communicator
from ..models.workloads import gradient_like, uniform_pm1
from ..ops.codecs import wire_ratio


def timed(fn, iters, warmup, world, dev, flush=None):
    for _ in range(warmup):
        fn()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    tot = 0.0
    if flush is None:
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(iters):
            fn()
        e.record()
        torch.cuda.synchronize()
        tot = s.elapsed_time(e)
    else:  # small messages: flush L2 between iterations, time each call, report the median
        each = []
        for _ in range(iters):
            flush.add_(1.0)
            if world > 1:
                dist.barrier()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            fn()
            e.record()
            torch.cuda.synchronize()
            each.append(s.elapsed_time(e))
        tot = sorted(each)[len(each) // 2] * iters   # a single 300 us hiccup would swamp a 30 us mean
    t = torch.tensor([tot / iters], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item() * 1e3  # us


def done_keys(csv_path: str, nranks: int, dtype: str) -> set:
    """(msg_size, algo, codec) of the rows a result CSV already holds for this job shape:
    what --resume skips, so that an interrupted sweep continues where it stopped."""
    keys = set()
    if not csv_path or not os.path.exists(csv_path):
        return keys
    with open(csv_path) as f:
        for line in f:
            p = line.strip().split(",")
            if len(p) >= 6 and p[0].isdigit() and p[1] == str(nranks) and p[2] == dtype:
                keys.add((int(p[0]), p[3], p[4]))
    return keys


def variant_key(var: str):
    """(algo column, codec column) of a --variants entry, as the rows print them."""
    parts = var.split(":")
    if parts[0] == "nccl":
        return "nccl", "none"
    algo = parts[1] if len(parts) > 1 else "auto"
    return algo + "".join(":" + q for q in parts[2:]), parts[0]


def main(argv=None):
    ap = argparse.ArgumentParser()
    # the long names are the ones to use under torch.distributed.run, whose own parser
    # takes a bare --max for an abbreviation of --max-restarts
    ap.add_argument("--min", "--min-bytes", dest="min", type=int, default=8)
    ap.add_argument("--max", "--max-bytes", dest="max", type=int, default=1 << 30)
    ap.add_argument("--factor", type=int, default=2)
    ap.add_argument("--sizes", default="", help="comma-separated byte sizes (overrides min/max)")
    ap.add_argument("--dtype", default="bf16")
    ap.add_argument("--data", default="uniform", choices=["uniform", "grad"])
    ap.add_argument("--variants", default="none:auto,int8:auto,nccl",
                    help="codec:algo[:waves[:ctas]] entries, or 'nccl'")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--arena-mb", type=int, default=2048)
    ap.add_argument("--csv", default="")
    ap.add_argument("--resume", action="store_true", help="skip the (size, algorithm, codec) rows already in --csv")
    ap.add_argument("--flush-below", type=int, default=64 << 20,
                    help="messages smaller than this are timed per call with an L2 flush in between")
    args = ap.parse_args(argv)

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    lr = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(lr)
    dev = torch.device("cuda", lr)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        comm = Communicator.from_torch_distributed(arena_bytes=args.arena_mb << 20, nvls=True)
    else:
        comm = Communicator.create(0, 1, f"sweep{os.getpid()}", arena_bytes=args.arena_mb << 20)
    dtype = {"bf16": torch.bfloat16, "f32": torch.float32, "f16": torch.float16}[args.dtype]
    es = torch.empty((), dtype=dtype).element_size()
    if args.sizes:
        sizes = [int(s) for s in args.sizes.split(",")]
    else:
        sizes, s = [], args.min
        while s <= args.max:
            sizes.append(s)
            s *= args.factor
    flush = torch.zeros(160 << 20, dtype=torch.float32, device=dev)  # 640 MB > L2
    rows = []
    done = done_keys(args.csv, world, args.dtype) if args.resume else set()
    header = "msg_size,nranks,dtype,algo,codec,time_us,algbw,busbw,ref_bw,ratio,rel_l2"
    if rank == 0:
        print(header, flush=True)
    for size in sizes:
        count = max(1, size // es)
        gen = gradient_like if args.data == "grad" else uniform_pm1
        x = gen(count, dtype, seed=rank, device=dev)
        y = torch.empty_like(x)
        exact = x.float().clone()
        if world > 1:
            dist.all_reduce(exact)
        for var in args.variants.split(","):
            if (count * es, *variant_key(var)) in done:   # every rank reads the same file: same decision everywhere
                continue
            parts = var.split(":")
            if parts[0] == "nccl":
                if world == 1:
                    continue
                codec, algo = "none", "nccl"

                def fn():
                    y.copy_(x)
                    dist.all_reduce(y)

                def fn_copy():
                    y.copy_(x)

                fl = flush if size < args.flush_below else None
                t = timed(fn, args.iters, args.warmup, world, dev, fl) - timed(fn_copy, args.iters, args.warmup, world, dev, fl)
                fn()  # leave the collective's result in y for the error column
            else:
                codec, algo = parts[0], parts[1] if len(parts) > 1 else "auto"
                comm.set_waves(int(parts[2]) if len(parts) > 2 else 0)
                comm.set_max_ctas(int(parts[3]) if len(parts) > 3 else 0)
                if algo in ("nvls", "nvls_inplace") and not comm.has_nvls:
                    continue
                if algo == "nvls_inplace":
                    # symmetric (arena-backed) tensor, reduced in place through the switch; the
                    # values grow from call to call, which does not change the time
                    if count * es > comm.arena_bytes // 2:
                        continue
                    xs = comm.symmetric_empty(count, dtype)
                    xs.copy_(x)

                    def fn():
                        comm.all_reduce(xs, codec="none", algo="nvls")

                    t = timed(fn, args.iters, args.warmup, world, dev, flush if size < args.flush_below else None)
                    xs.copy_(x)
                    fn()
                    y.copy_(xs)
                    del xs
                    comm.symmetric_free_all()
                    if comm.status()[0] != 0:
                        raise SystemExit(f"communicator failed: {comm.status()}")
                    rel = ((y.float() - exact).norm() / (exact.norm() + 1e-30)).item()
                    bytes_ = count * es
                    algbw = bytes_ / (t * 1e-6) / 1e9
                    bus = algbw * (2 * (world - 1) / world if world > 1 else 1.0)
                    row = f"{bytes_},{world},{args.dtype},nvls_inplace,none,{t:.2f},{algbw:.2f},{bus:.2f},{2 * algbw:.2f},1.000,{rel:.3e}"
                    rows.append(row)
                    if rank == 0:
                        print(row, flush=True)
                    continue

                def fn():
                    comm.all_reduce(x, y, codec=codec, algo=algo)

                t = timed(fn, args.iters, args.warmup, world, dev, flush if size < args.flush_below else None)
                if comm.status()[0] != 0:
                    raise SystemExit(f"communicator failed: {comm.status()}")
            rel = ((y.float() - exact).norm() / (exact.norm() + 1e-30)).item()
            bytes_ = count * es
            algbw = bytes_ / (t * 1e-6) / 1e9
            bus = algbw * (2 * (world - 1) / world if world > 1 else 1.0)
            name = algo + ("".join(":" + p for p in parts[2:]) if len(parts) > 2 else "")
            row = f"{bytes_},{world},{args.dtype},{name},{codec},{t:.2f},{algbw:.2f},{bus:.2f},{2 * algbw:.2f},{wire_ratio(codec, dtype):.3f},{rel:.3e}"
            rows.append(row)
            if rank == 0:
                print(row, flush=True)
        del x, y, exact
    if rank == 0 and args.csv:
        new = not os.path.exists(args.csv)
        os.makedirs(os.path.dirname(os.path.abspath(args.csv)), exist_ok=True)
        with open(args.csv, "a") as f:
            if new:
                f.write(header + "\n")
            f.write("\n".join(rows) + "\n")
    comm.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
