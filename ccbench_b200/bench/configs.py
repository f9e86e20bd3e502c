"""Benchmarks of the named configurations 3, 4 and 5 (1..8 GPUs, one process per GPU
under torch.distributed.run), each against the plain NCCL call timed the same way.
All times are CUDA-event times on the device, maximum over ranks, after warm-up.

    python -m torch.distributed.run --nproc-per-node N -m ccbench_b200.bench.configs --config 3
    ... --config 4 [--field 512]      error-bounded AllGather / Broadcast of a smooth field
    ... --config 5                    MoE dispatch/combine (fp8) and bucketed int8 ReduceScatter on a side stream

Bus bandwidth uses the nccl-tests factors: AllReduce 2(n-1)/n, AllGather /
ReduceScatter / AlltoAll (n-1)/n, Broadcast 1."""
from __future__ import annotations

import argparse
import json
import math
import os

import torch
import torch.distributed as dist

from .. import Communicator
from ..models.workloads import gradient_like, moe_routing, normal, smooth_field
from ..ops import sz
from ..ops.codecs import wire_ratio
from ..parallel import moe


def _timed(fn, iters, warmup, world, dev):
    for _ in range(warmup):
        fn()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(iters):
        fn()
    e.record()
    torch.cuda.synchronize()
    t = torch.tensor([s.elapsed_time(e) / iters], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item() * 1e3  # us


def _emit(rank, row):
    if rank == 0:
        print(json.dumps(row), flush=True)


def config3(comm, rank, world, dev, args):
    dtype = torch.bfloat16
    count = args.bytes // 2
    x = gradient_like(count, dtype, seed=rank, device=dev)
    y = torch.empty_like(x)
    exact = x.float().clone()
    if world > 1:
        dist.all_reduce(exact)
    f = 2 * (world - 1) / world if world > 1 else 1.0
    for algo in ("twoshot", "ring", "tree"):
        for codec in ("int8", "fp8"):
            for ef_on in (False, True):
                ef = torch.zeros(count, device=dev) if ef_on else None
                fn = lambda: comm.all_reduce(x, y, codec=codec, algo=algo, error_feedback=ef)
                t = _timed(fn, args.iters, args.warmup, world, dev)
                assert comm.status()[0] == 0
                rel1 = ((y.float() - exact).norm() / exact.norm()).item()
                rel_avg = None
                if ef_on:  # what error feedback buys: the error of the running mean of the results
                    ef.zero_()
                    acc = torch.zeros(count, device=dev)
                    for _ in range(8):
                        fn()
                        acc += y.float()
                    rel_avg = ((acc / 8 - exact).norm() / exact.norm()).item()
                _emit(rank, {"config": 3, "algo": algo, "codec": codec, "error_feedback": ef_on, "n": world, "bytes": args.bytes,
                             "time_us": round(t, 2), "busbw_GBs": round(args.bytes / t / 1e3 * f, 2), "ratio": round(wire_ratio(codec, dtype), 3),
                             "rel_l2": rel1, "rel_l2_mean_of_8": rel_avg})
                del ef
    if world > 1:
        z = x.clone()
        t = _timed(lambda: dist.all_reduce(z), args.iters, args.warmup, world, dev)
        _emit(rank, {"config": 3, "algo": "nccl", "codec": "none", "n": world, "bytes": args.bytes, "time_us": round(t, 2),
                     "busbw_GBs": round(args.bytes / t / 1e3 * f, 2), "ratio": 1.0})


def config4(comm, rank, world, dev, args):
    n = args.field
    fld = smooth_field(n, seed=rank, device=dev)
    rng = (fld.max() - fld.min()).item()
    eb = 1e-4 * rng
    raw = fld.numel() * 4
    recv = torch.empty((world, n, n, n), device=dev)
    used = torch.zeros(1, dtype=torch.int64, device=dev)
    t = _timed(lambda: sz.all_gather(comm, fld, recv, eb, used), args.iters, args.warmup, world, dev)
    assert comm.status()[0] == 0
    err = (recv[rank] - fld).abs().max().item()
    mse = ((recv[rank] - fld).double() ** 2).mean().item()
    ratio = raw / max(int(used.item()), 1)
    fa = (world - 1) / world if world > 1 else 1.0
    _emit(rank, {"config": 4, "op": "allgather", "codec": "ccb-sz v2", "n": world, "field": n, "raw_bytes_per_rank": raw, "eb": eb,
                 "time_us": round(t, 2), "busbw_GBs": round(raw * world / t / 1e3 * fa, 2), "ratio": round(ratio, 3),
                 "max_err": err, "bound_held": err <= float(torch.tensor(eb, dtype=torch.float32)), "psnr_dB": 20 * math.log10(rng) - 10 * math.log10(mse)})
    out = torch.empty_like(fld)
    t = _timed(lambda: sz.broadcast(comm, fld, out, eb, root=0, used=used), args.iters, args.warmup, world, dev)
    assert comm.status()[0] == 0
    _emit(rank, {"config": 4, "op": "broadcast", "codec": "ccb-sz v2", "n": world, "field": n, "time_us": round(t, 2),
                 "busbw_GBs": round(raw / t / 1e3, 2)})
    if world > 1:
        t = _timed(lambda: dist.all_gather_into_tensor(recv.view(-1), fld.view(-1)), args.iters, args.warmup, world, dev)
        _emit(rank, {"config": 4, "op": "allgather", "codec": "none (nccl)", "n": world, "time_us": round(t, 2),
                     "busbw_GBs": round(raw * world / t / 1e3 * fa, 2), "ratio": 1.0})
        t = _timed(lambda: dist.broadcast(out, 0), args.iters, args.warmup, world, dev)
        _emit(rank, {"config": 4, "op": "broadcast", "codec": "none (nccl)", "n": world, "time_us": round(t, 2), "busbw_GBs": round(raw / t / 1e3, 2)})
    # codec alone (one GPU's view): compress and decompress throughput
    buf, used1 = sz.compress(fld, eb)
    tc = _timed(lambda: sz.compress(fld, eb), args.iters, args.warmup, 1, dev)
    td = _timed(lambda: sz.decompress(buf, fld.shape, eb), args.iters, args.warmup, 1, dev)
    _emit(rank, {"config": 4, "op": "codec only", "compress_GBs": round(raw / tc / 1e3, 1), "decompress_GBs": round(raw / td / 1e3, 1)})


def config5(comm, rank, world, dev, args):
    T, H, K = args.tokens, args.hidden, 2
    dt = torch.bfloat16
    x = normal(T * H, dt, seed=rank, device=dev).view(T, H)
    ids, gates = moe_routing(T, world, K, seed=rank, device=dev)
    route = moe.plan_route(ids, gates, world)
    counts = [torch.zeros_like(route.send_counts) for _ in range(world)]
    if world > 1:
        dist.all_gather(counts, route.send_counts)
    else:
        counts = [route.send_counts]
    cm = [c.tolist() for c in counts]
    rows_in = sum(cm[s][rank] for s in range(world))
    recv = torch.empty(max(rows_in, 1), H, dtype=dt, device=dev)
    out = torch.empty(T, H, dtype=dt, device=dev)
    fa = (world - 1) / world if world > 1 else 1.0
    sent = T * K * H * 2
    for codec in ("fp8", "none"):
        td = _timed(lambda: moe.dispatch(comm, x, recv, route, cm, codec=codec), args.iters, args.warmup, world, dev)
        tcmb = _timed(lambda: moe.combine(comm, recv, out, route, cm, codec=codec), args.iters, args.warmup, world, dev)
        assert comm.status()[0] == 0
        _emit(rank, {"config": 5, "op": "moe dispatch+combine", "codec": codec, "n": world, "tokens": T, "hidden": H, "topk": K,
                     "dispatch_us": round(td, 2), "combine_us": round(tcmb, 2), "dispatch_busbw_GBs": round(sent / td / 1e3 * fa, 2),
                     "combine_busbw_GBs": round(sent / tcmb / 1e3 * fa, 2), "ratio": round(wire_ratio(codec, dt), 3)})
    if world > 1:  # NCCL baseline: equal-split all_to_all of the same volume (+ the permute it needs)
        send_sorted = x[route.perm.long()]
        in_split = route.send_counts.tolist()
        out_split = [cm[s][rank] for s in range(world)]

        def nccl_dispatch():
            s = x[route.perm.long()]
            dist.all_to_all_single(recv[:rows_in], s, out_split, in_split)

        t = _timed(nccl_dispatch, args.iters, args.warmup, world, dev)
        _emit(rank, {"config": 5, "op": "moe dispatch", "codec": "none (nccl all_to_all + gather kernel)", "n": world, "dispatch_us": round(t, 2),
                     "dispatch_busbw_GBs": round(sent / t / 1e3 * fa, 2)})
        del send_sorted
    # ZeRO-style gradient buckets: 40 x 25 MiB bf16, int8 ReduceScatter on a side stream under a compute stream
    bucket = (25 << 20) // 2
    bucket -= bucket % (world * 512)
    g = gradient_like(bucket, dt, seed=rank, device=dev)
    shard = torch.empty(bucket // world, dtype=dt, device=dev)
    nb = args.buckets
    # high priority: the collective's CTAs take the first SMs a GEMM wave frees, instead of queueing behind it
    side = torch.cuda.Stream(priority=-1)
    a = torch.randn(8192, 8192, device=dev, dtype=dt)

    def comm_only():
        for _ in range(nb):
            comm.reduce_scatter(g, shard, codec="int8")

    def nccl_only():
        for _ in range(nb):
            dist.reduce_scatter_tensor(shard, g)

    def compute_only():
        for _ in range(nb):
            torch.matmul(a, a)

    def both(comm_fn):
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            comm_fn()
        compute_only()
        torch.cuda.current_stream().wait_stream(side)

    t_comp = _timed(compute_only, 3, 1, world, dev)
    # The collective kernel is one co-resident grid: with every SM taken it starves the GEMMs
    # it should hide behind, so the grid is capped and the cap swept (0 = no cap).
    for cap, plain in ((0, False), (64, False), (32, False), (32, True), (16, True), (8, True)):
        comm.set_max_ctas(cap)
        comm.set_noncooperative(cap if plain else 0)
        t_comm = _timed(comm_only, 3, 1, world, dev)
        t_both = _timed(lambda: both(comm_only), 3, 1, world, dev)
        assert comm.status()[0] == 0
        _emit(rank, {"config": 5, "op": "reduce_scatter buckets", "codec": "int8", "n": world, "buckets": nb, "bucket_bytes": bucket * 2,
                     "max_ctas": cap, "launch": "plain" if plain else "cooperative", "comm_alone_us": round(t_comm, 1), "compute_alone_us": round(t_comp, 1),
                     "overlapped_us": round(t_both, 1), "busbw_GBs": round(bucket * 2 * nb / t_comm / 1e3 * fa, 2),
                     "exposed_comm_us": round(t_both - t_comp, 1),
                     "overlap_efficiency": round((t_comm + t_comp - t_both) / min(t_comm, t_comp), 3)})
    comm.set_max_ctas(0)
    comm.set_noncooperative(0)
    if world > 1:
        t_nccl = _timed(nccl_only, 3, 1, world, dev)
        t_both = _timed(lambda: both(nccl_only), 3, 1, world, dev)
        _emit(rank, {"config": 5, "op": "reduce_scatter buckets", "codec": "none (nccl)", "n": world, "buckets": nb,
                     "bucket_bytes": bucket * 2, "comm_alone_us": round(t_nccl, 1), "compute_alone_us": round(t_comp, 1),
                     "overlapped_us": round(t_both, 1), "busbw_GBs": round(bucket * 2 * nb / t_nccl / 1e3 * fa, 2),
                     "exposed_comm_us": round(t_both - t_comp, 1),
                     "overlap_efficiency": round((t_nccl + t_comp - t_both) / min(t_nccl, t_comp), 3)})


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", type=int, required=True, choices=[3, 4, 5])
    ap.add_argument("--bytes", type=int, default=256 << 20)
    ap.add_argument("--field", type=int, default=512)
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--buckets", type=int, default=40)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--arena-mb", type=int, default=0)
    a = ap.parse_args(argv)
    world, rank, lr = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(lr)
    dev = torch.device("cuda", lr)
    arena = a.arena_mb << 20
    if not arena and a.config == 4:
        arena = 2 * world * sz.capacity((a.field,) * 3) + (64 << 20)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        comm = Communicator.from_torch_distributed(arena_bytes=arena, nvls=os.environ.get("CCB_NVLS", "1") == "1")
    else:
        comm = Communicator.create(0, 1, f"cfg{os.getpid()}", arena_bytes=arena)
    {3: config3, 4: config4, 5: config5}[a.config](comm, rank, world, dev, a)
    comm.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
