"""MoE dispatch / combine: routed token exchange with per-destination compression,
all ranks played on one GPU, against a plain torch restatement."""
import pytest
import torch

from ccbench_b200 import Communicator
from ccbench_b200.models.workloads import moe_routing
from ccbench_b200.ops import codecs as C
from ccbench_b200.parallel import moe

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("codec", ["fp8", "none", "int8"])
@pytest.mark.parametrize("n,T,H", [(4, 300, 1024), (8, 256, 512), (2, 77, 2048)])
def test_dispatch_then_combine(codec, n, T, H):
    comm = Communicator.local(n, arena_bytes=64 << 20)
    try:
        dt = torch.bfloat16
        xs = [torch.randn(T, H, generator=torch.Generator().manual_seed(r)).to(dt) for r in range(n)]
        routes_cpu = []
        for r in range(n):
            ids, gates = moe_routing(T, n, 2, seed=r)
            routes_cpu.append(moe.plan_route(ids, gates, n))
        cm = [rt.send_counts.tolist() for rt in routes_cpu]
        to_dev = lambda rt: moe.Route(rt.perm.cuda(), rt.dest_rank.cuda(), rt.pos.cuda(), rt.gate.cuda(), rt.send_counts, rt.topk)
        routes = [to_dev(rt) for rt in routes_cpu]
        xg = [x.cuda() for x in xs]
        rows_in = [sum(cm[s][d] for s in range(n)) for d in range(n)]
        recv = [torch.zeros(max(rows_in[d], 1), H, dtype=dt, device="cuda") for d in range(n)]
        for _ in range(2):
            moe.dispatch(comm, xg, recv, routes, cm, codec=codec)
        torch.cuda.synchronize()
        assert comm.status()[0] == 0
        rt_ = lambda v: C.roundtrip(v.float(), codec, dt).to(dt)
        for d in range(n):
            want = []
            for s in range(n):
                rtc = routes_cpu[s]
                start = sum(cm[s][:d])
                rows = rtc.perm[start:start + cm[s][d]].long()
                want.append(rt_(xs[s][rows]).reshape(-1, H))
            want = torch.cat(want) if want else torch.zeros(0, H, dtype=dt)
            assert torch.equal(recv[d][:rows_in[d]].cpu(), want)
        # experts scale their inputs; combine brings them back gate-weighted
        ys = [(recv[d].float() * (d + 1)).to(dt) for d in range(n)]
        out = [torch.zeros(T, H, dtype=dt, device="cuda") for _ in range(n)]
        moe.combine(comm, ys, out, routes, cm, codec=codec)
        torch.cuda.synchronize()
        assert comm.status()[0] == 0
        for s in range(n):
            rtc = routes_cpu[s]
            acc = torch.zeros(T, H)
            for pair in range(T * 2):
                t, d, j = pair // 2, int(rtc.dest_rank[pair]), int(rtc.pos[pair])
                row0 = sum(cm[q][d] for q in range(s))
                acc[t] += rtc.gate[pair] * rt_(ys[d][row0 + j].cpu()).float()
            got = out[s].float().cpu()
            assert (got - acc).abs().max().item() <= 2.0 ** -7 * acc.abs().max().item() + 1e-6
    finally:
        comm.close()
