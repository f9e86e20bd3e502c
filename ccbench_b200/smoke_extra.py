"""Extra one-step checks run by smoke(): one launch of every other kernel family on
cuda:0, each compared with a plain PyTorch statement of the same operation. Inputs are
generated on the CPU and copied, so that the kernels launched here are this library's
(the error-bounded codec, MoE dispatch / combine, the exchange and reduce families, the
pipelined two-shot kernel, the lossless codec) and not input generation."""
import torch


def run() -> None:
    from . import Communicator
    from .models.workloads import moe_routing, smooth_field
    from .ops import codecs as C
    from .ops import sz
    from .parallel import moe

    dev = torch.device("cuda", 0)
    n = 4
    comm = Communicator.local(n, arena_bytes=48 << 20)
    try:
        # error-bounded codec: local round trip and the fused all-gather
        f = [smooth_field(40, seed=r, device="cpu").to(dev) for r in range(n)]
        eb = 1e-3 * (f[0].max() - f[0].min()).item()
        buf, used = sz.compress(f[0], eb)
        back = sz.decompress(buf, f[0].shape, eb)
        eb32 = float(torch.tensor(eb, dtype=torch.float32))
        assert (back - f[0]).abs().max().item() <= eb32 and 0 < int(used.item()) < f[0].numel() * 4
        recv = [torch.empty((n,) + tuple(f[0].shape), device=dev) for _ in range(n)]
        sz.all_gather(comm, f, recv, eb)
        torch.cuda.synchronize()
        assert torch.equal(recv[3][0], back)
        assert max((recv[1][q] - f[q]).abs().max().item() for q in range(n)) <= eb32

        # MoE dispatch with fp8 rows, then combine with identity experts
        T, H, dt = 128, 1024, torch.bfloat16
        tok = [torch.randn(T, H, generator=torch.Generator().manual_seed(10 + r)).to(dt).to(dev) for r in range(n)]
        routes = [moe.plan_route(*(t.to(dev) for t in moe_routing(T, n, 2, seed=r, device="cpu")), n) for r in range(n)]
        cm = [rt.send_counts.tolist() for rt in routes]
        rows = [max(sum(cm[s][d] for s in range(n)), 1) for d in range(n)]
        got = [torch.zeros(rows[d], H, dtype=dt, device=dev) for d in range(n)]
        moe.dispatch(comm, tok, got, routes, cm, codec="fp8")
        out = [torch.zeros(T, H, dtype=dt, device=dev) for _ in range(n)]
        moe.combine(comm, got, out, routes, cm, codec="fp8")
        torch.cuda.synchronize()
        rel = ((out[0].float() - tok[0].float()).norm() / tok[0].float().norm()).item()
        assert rel < 0.15, rel

        # exchange family: all-gather with fp8 lanes, all-to-all verbatim
        per = 4096 + 3
        xs = [torch.randn(per * n, generator=torch.Generator().manual_seed(r)) for r in range(n)]
        xg = [x.to(dev) for x in xs]
        ag = [torch.empty(per * n * n, device=dev) for _ in range(n)]
        comm.all_gather(xg, ag, codec="fp8")
        a2a = [torch.empty(per * n, device=dev) for _ in range(n)]
        comm.all_to_all(xg, a2a, codec="none")
        torch.cuda.synchronize()
        assert torch.equal(ag[1].cpu(), torch.cat([C.roundtrip(x, "fp8") for x in xs]))
        assert torch.equal(a2a[2].cpu(), torch.cat([x[2 * per:3 * per] for x in xs]))

        # reduce-scatter with int8 lanes
        rs = [torch.empty(per, device=dev) for _ in range(n)]
        comm.reduce_scatter(xg, rs, codec="int8")
        torch.cuda.synchronize()
        exact = sum(x[per:2 * per].double() for x in xs).float()
        assert ((rs[1].cpu() - exact).norm() / exact.norm()).item() < 0.03

        # the warp-specialised pipelined two-shot kernel, forced on for a small message
        comm.set_pipeline(2)
        comm.set_waves(2)
        ys = [torch.randn(50000, generator=torch.Generator().manual_seed(40 + r)).to(torch.bfloat16) for r in range(n)]
        yg = [y.to(dev) for y in ys]
        yo = [torch.empty_like(y) for y in yg]
        comm.all_reduce(yg, yo, codec="int8", algo="twoshot")
        comm.set_pipeline(1)
        comm.set_waves(0)
        torch.cuda.synchronize()
        exact = sum(y.double() for y in ys).float()
        assert ((yo[2].float().cpu() - exact).norm() / exact.norm()).item() < 0.03

        # lossless float codec: bit-exact round trip
        from .ops import lossless

        z = (torch.randn(10000, generator=torch.Generator().manual_seed(7)) * 1e-3).to(torch.bfloat16).to(dev)
        comp = lossless.encode(z)
        assert torch.equal(lossless.decode(comp, z.numel(), z.dtype), z)
        assert lossless.used_bytes(comp) < z.numel() * 2
        assert comm.status()[0] == 0
    finally:
        comm.close()
    # the link probe (stores and bulk copies into the own arena on a one-rank communicator)
    # and the integer fold of the NCCL-free provider
    import ctypes
    import os

    from ._lib import lib
    from .comm import _check

    one = Communicator.create(0, 1, f"smoke{os.getpid()}", arena_bytes=64 << 20)
    try:
        stream = torch.cuda.current_stream().cuda_stream
        for method in (0, 2):
            _check(lib().ccb_link_probe(one._h, method, 0, 8 << 20, stream))
        parts = torch.arange(3 * 1000, dtype=torch.int32).reshape(3, 1000).to(dev)
        out = torch.empty(1000, dtype=torch.int32, device=dev)
        _check(lib().ccb_fold(18, 0, ctypes.c_void_p(parts.data_ptr()), 1000, 3, 1000, ctypes.c_void_p(out.data_ptr()), stream))
        torch.cuda.synchronize()
        assert torch.equal(out, parts.sum(0).to(torch.int32)) and one.status()[0] == 0
    finally:
        one.close()
