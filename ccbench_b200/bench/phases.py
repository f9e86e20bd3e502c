"""Phase timeline of the fused kernels from their own per-CTA timestamps
(`Communicator.set_trace`): where inside ONE launch the time goes. No profiler involved;
the marks are `globaltimer` reads by thread 0 of every CTA.

    python -m torch.distributed.run --nproc-per-node 4 -m ccbench_b200.bench.phases --what allreduce
    python -m torch.distributed.run --nproc-per-node 4 -m ccbench_b200.bench.phases --what sz --field 384

allreduce (two-shot): marks 0 start, 1 own lanes pushed to the owners, 3 own shard reduced,
re-encoded and pushed to everybody, 4 all shards decoded. Large messages run the
warp-specialised pipelined kernel; its row gives mark 1 = first wave's lanes pushed (all
warps), 2 = first wave reduced by the link warps, 3 = link warps done, 5 = first wave
decoded, 4 = decode warps done, then the time the link leader waited for flags and the
time the signal warp spent in fences; the row "plain" is the same call with the pipelined
kernel switched off. sz: 0 start, 1 own field packed
and copied out, 3 first received field decoded, 4 all decoded. Times are microseconds
after the first CTA of the rank started, median / max over the CTAs.
"""
from __future__ import annotations

import argparse
import os

import torch
import torch.distributed as dist

from .. import Communicator
from ..models.workloads import gradient_like, smooth_field
from ..ops import sz


def _timed(fn, world, dev, iters=10):
    ts = []
    for _ in range(iters):
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        ts.append(s.elapsed_time(e) * 1e3)
    t = torch.tensor([sorted(ts)[len(ts) // 2]], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()


def _trace(comm, fn, world, marks, extra=False):
    comm.set_trace(True)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    fn()
    torch.cuda.synchronize()
    tr = comm.read_trace(1024).double()   # before tracing is switched off: that releases the marks
    comm.set_trace(False)
    tr = tr[tr[:, 0] > 0]
    rel = (tr - tr[:, 0].min()) / 1e3
    line = f"ctas {tr.shape[0]} | " + " | ".join(f"mark {k}: {rel[:, k].median():.1f} / {rel[:, k].max():.1f}" for k in marks)
    if extra:
        line += f" | waited {tr[:, 6].median() / 1e3:.1f} / {tr[:, 6].max() / 1e3:.1f} | in fences {tr[:, 7].median() / 1e3:.1f} / {tr[:, 7].max() / 1e3:.1f}"
    return line


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--what", default="allreduce", choices=["allreduce", "sz"])
    ap.add_argument("--codec", default="int8")
    ap.add_argument("--field", type=int, default=384)
    a = ap.parse_args(argv)
    world, rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))
    lr = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(lr)
    dev = torch.device("cuda", lr)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    if a.what == "allreduce":
        comm = Communicator.from_torch_distributed() if world > 1 else Communicator.create(0, 1, f"ph{os.getpid()}")
        for dt, nbytes in [(torch.float32, 1 << 20), (torch.float32, 16 << 20), (torch.bfloat16, 256 << 20)]:
            count = nbytes // torch.empty((), dtype=dt).element_size()
            x = gradient_like(count, dt, seed=rank, device=dev)
            y = torch.empty_like(x)
            for algo in ("twoshot", "oneshot", "ring"):
                if algo == "oneshot" and nbytes > (64 << 20):
                    continue
                fn = lambda: comm.all_reduce(x, y, codec=a.codec, algo=algo)
                for _ in range(5):
                    fn()
                line = f"n={world} {nbytes >> 20} MiB {a.codec} {algo}: {_timed(fn, world, dev):.1f} us"
                big = algo == "twoshot" and world > 1 and nbytes >= (64 << 20)
                if algo == "twoshot":
                    line += " | " + (_trace(comm, fn, world, (1, 2, 3, 5, 4), extra=True) if big else _trace(comm, fn, world, (1, 3, 4)))
                if rank == 0:
                    print(line, flush=True)
                if big:
                    comm.set_pipeline(0)
                    for _ in range(3):
                        fn()
                    line = f"n={world} {nbytes >> 20} MiB {a.codec} twoshot plain: {_timed(fn, world, dev):.1f} us | " + _trace(comm, fn, world, (1, 3, 4))
                    comm.set_pipeline(1)
                    if rank == 0:
                        print(line, flush=True)
            if world > 1:
                z = x.clone()
                for _ in range(5):
                    dist.all_reduce(z)
                t = _timed(lambda: dist.all_reduce(z), world, dev)
                if rank == 0:
                    print(f"n={world} {nbytes >> 20} MiB nccl: {t:.1f} us", flush=True)
    else:
        n = a.field
        arena = 2 * world * sz.capacity((n,) * 3) + (64 << 20)
        nvls = os.environ.get("CCB_NVLS", "1") == "1"
        comm = (Communicator.from_torch_distributed(arena_bytes=arena, nvls=nvls) if world > 1
                else Communicator.create(0, 1, f"ph{os.getpid()}", arena_bytes=arena))
        fld = smooth_field(n, seed=rank, device=dev)
        eb = 1e-4 * (fld.max() - fld.min()).item()
        recv = torch.empty((world, n, n, n), device=dev)
        out = torch.empty_like(fld)
        for name, fn in (("all-gather", lambda: sz.all_gather(comm, fld, recv, eb)),
                         ("broadcast", lambda: sz.broadcast(comm, fld, out, eb, root=0))):
            for _ in range(3):
                fn()
            t = _timed(fn, world, dev, 5)
            msg = f"sz {name} n={world} field {n}^3: {t:.1f} us | rank {rank} " + _trace(comm, fn, world, (1, 3, 4))
            for q in range(min(world, 2)):   # the root and one receiver
                if rank == q:
                    print(msg, flush=True)
                if world > 1:
                    dist.barrier()
    comm.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
