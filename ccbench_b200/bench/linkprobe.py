"""Peer-store bandwidth by store method: the link roofline of the fused collectives.

    python -m torch.distributed.run --nproc-per-node 2 -m ccbench_b200.bench.linkprobe

Every rank writes into the arena of rank + 1 (all at once: every link carries traffic in
both directions, as in a collective), then rank 0 alone (one direction). Methods: 16-byte
stores per lane, bulk copies of 512 bytes and of 2 KB from shared memory (TMA unit), and
torch's peer copy (copy engine) for reference. Device-timed, max over ranks."""
from __future__ import annotations

import argparse
import os

import torch
import torch.distributed as dist

from .. import Communicator
from .._lib import lib
from ..comm import _check

METHODS = {0: "st.global.v4 per lane", 1: "bulk copy 512 B", 2: "bulk copy 2 KB"}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--bytes", type=int, default=256 << 20)
    ap.add_argument("--iters", type=int, default=10)
    a = ap.parse_args(argv)
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0)))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    comm = Communicator.from_torch_distributed(arena_bytes=(2 * a.bytes) + (256 << 20))
    peer = (rank + 1) % world
    stream = torch.cuda.current_stream().cuda_stream

    def timed(fn, active):
        for _ in range(3):
            if active:
                fn()
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(a.iters):
            if active:
                fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / a.iters if active else 0.0], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item() * 1e-3

    for both in (True, False):
        for m, name in METHODS.items():
            s = timed(lambda: _check(lib().ccb_link_probe(comm._h, m, peer, a.bytes, stream)), both or rank == 0)
            if rank == 0:
                print(f"{'all ranks' if both else 'rank 0 only':12s} {name:24s} {a.bytes / s / 1e9:8.1f} GB/s per direction ({s * 1e6:.1f} us)", flush=True)
    assert comm.status()[0] == 0
    comm.close()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
