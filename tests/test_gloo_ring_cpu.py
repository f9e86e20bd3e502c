"""The CPU ring over torch.distributed gloo equals the restated ring algorithm bit for bit."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from ccbench_b200.bench import config1_gloo
from ccbench_b200.ops import codecs as C


def _worker(rank, world, port, count, codec, q):
    from ccbench_b200.parallel.cpu_ring import ring_all_reduce

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.set_num_threads(1)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    x = torch.randn(count, generator=torch.Generator().manual_seed(100 + rank)) * (rank + 1)
    y = ring_all_reduce(x, codec)
    # plain bytes, not a tensor: a tensor travels through a shared-memory handshake with this
    # process, which may already have exited when the parent asks for it
    q.put((rank, y.numpy().tobytes()))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world,count,codec", [(2, 5000, "int8"), (3, 4099, "int8"), (4, 70001, "fp8"), (3, 1000, "none")])
def test_ring_matches_the_restatement(world, count, codec):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, count, codec, q)) for r in range(world)]
    for p in procs:
        p.start()
    import numpy as np

    got = {r: torch.from_numpy(np.frombuffer(b, dtype=np.float32).copy()) for r, b in (q.get(timeout=300) for _ in range(world))}
    for p in procs:
        p.join(timeout=60)
    xs = [torch.randn(count, generator=torch.Generator().manual_seed(100 + r)) * (r + 1) for r in range(world)]
    want = C.simulate_all_reduce(xs, codec, "ring", torch.float32)
    for r in range(world):
        assert torch.equal(got[r], want), (r, (got[r] - want).abs().max())


def test_configuration_1_over_gloo():
    res = config1_gloo.run(ranks=2, elements=1 << 16, iters=2)
    assert res["uncompressed"]["rel_l2"] < 1e-6
    q = res["int8_block"]
    assert 0 < q["rel_l2"] < 0.02 and abs(q["compression_ratio"] - 4 / (1 + 4 / 128)) < 0.01
    assert q["latency_us_max_over_ranks"] > 0
