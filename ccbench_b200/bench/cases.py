"""Small single-GPU cases of the hot kernels, sized for a profiler capture: inputs
larger than L2 (126 MB) but well under a few GB, a few launches, no multi-rank
process. `python -m ccbench_b200.bench.cases --case NAME [--launches 3]`.

  allreduce_int8_1rank   two-shot kernel on one rank: the codec round trip at HBM speed
  allreduce_int8_8ranks  eight ranks played on this GPU by one cooperative launch
  sz_compress            error-bounded codec, 384^3 fp32 field (226 MB)
  sz_decompress
  moe_dispatch_fp8       4096 tokens x 4096 hidden bf16, 4 ranks on this GPU
  allreduce_ring_int8_8ranks   ring kernel, eight ranks on this GPU, 16 Mi bf16 each
  allgather_fp8_8ranks   exchange kernel, eight ranks on this GPU, 4 Mi bf16 each
  allreduce_pipe_int8_4ranks   warp-specialised two-shot kernel (1024 threads), four ranks on
                         this GPU, 16 Mi bf16 each
  lossless_encode / lossless_decode   lossless float codec, 128 Mi bf16 (256 MB)
"""
from __future__ import annotations

import argparse
import os

import torch

from .. import Communicator
from ..models.workloads import gradient_like, moe_routing, normal, smooth_field
from ..ops import sz
from ..parallel import moe


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", required=True)
    ap.add_argument("--launches", type=int, default=3)
    a = ap.parse_args(argv)
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    if a.case == "allreduce_int8_1rank":
        comm = Communicator.create(0, 1, f"case{os.getpid()}", arena_bytes=640 << 20)
        x = gradient_like(128 << 20, torch.bfloat16, device=dev)
        y = torch.empty_like(x)
        for _ in range(a.launches):
            comm.all_reduce(x, y, codec="int8", algo="twoshot")
    elif a.case == "allreduce_int8_8ranks":
        n = 8
        comm = Communicator.local(n, arena_bytes=96 << 20)
        xs = [gradient_like(16 << 20, torch.bfloat16, seed=r, device=dev) for r in range(n)]
        ys = [torch.empty_like(x) for x in xs]
        for _ in range(a.launches):
            comm.all_reduce(xs, ys, codec="int8", algo="twoshot")
    elif a.case == "allreduce_ring_int8_8ranks":
        n = 8
        comm = Communicator.local(n, arena_bytes=96 << 20)
        xs = [gradient_like(16 << 20, torch.bfloat16, seed=r, device=dev) for r in range(n)]
        ys = [torch.empty_like(x) for x in xs]
        for _ in range(a.launches):
            comm.all_reduce(xs, ys, codec="int8", algo="ring")
    elif a.case == "allreduce_pipe_int8_4ranks":
        n = 4
        comm = Communicator.local(n, arena_bytes=96 << 20)
        comm.set_pipeline(2)
        xs = [gradient_like(16 << 20, torch.bfloat16, seed=r, device=dev) for r in range(n)]
        ys = [torch.empty_like(x) for x in xs]
        for _ in range(a.launches):
            comm.all_reduce(xs, ys, codec="int8", algo="twoshot")
    elif a.case in ("lossless_encode", "lossless_decode"):
        from ..ops import lossless

        x = gradient_like(128 << 20, torch.bfloat16, device=dev)
        comp = lossless.encode(x)
        out = torch.empty_like(x)
        for _ in range(a.launches):
            if a.case == "lossless_encode":
                lossless.encode(x)
            else:
                lossless.decode(comp, x.numel(), x.dtype, out=out)
    elif a.case == "allgather_fp8_8ranks":
        n = 8
        comm = Communicator.local(n, arena_bytes=96 << 20)
        xs = [normal(4 << 20, torch.bfloat16, seed=r, device=dev) for r in range(n)]
        ys = [torch.empty(n * (4 << 20), dtype=torch.bfloat16, device=dev) for _ in range(n)]
        for _ in range(a.launches):
            comm.all_gather(xs, ys, codec="fp8")
    elif a.case in ("sz_compress", "sz_decompress"):
        f = smooth_field(384, device=dev)
        eb = 1e-4 * (f.max() - f.min()).item()
        buf, _ = sz.compress(f, eb)
        for _ in range(a.launches):
            if a.case == "sz_compress":
                sz.compress(f, eb)
            else:
                sz.decompress(buf, f.shape, eb)
    elif a.case == "moe_dispatch_fp8":
        n, T, H = 4, 4096, 4096
        comm = Communicator.local(n, arena_bytes=192 << 20)
        xs = [normal(T * H, torch.bfloat16, seed=r, device=dev).view(T, H) for r in range(n)]
        routes = [moe.plan_route(*moe_routing(T, n, 2, seed=r, device=dev), n) for r in range(n)]
        cm = [rt.send_counts.tolist() for rt in routes]
        recv = [torch.empty(sum(cm[s][d] for s in range(n)), H, dtype=torch.bfloat16, device=dev) for d in range(n)]
        for _ in range(a.launches):
            moe.dispatch(comm, xs, recv, routes, cm, codec="fp8")
    else:
        raise SystemExit(f"unknown case {a.case}")
    torch.cuda.synchronize()
    print("case", a.case, "done")


if __name__ == "__main__":
    main()
