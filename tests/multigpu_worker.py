"""Worker of the multi-GPU tests: one process per GPU under torch.distributed.run.
Checks every collective over real peer memory against torch.distributed (NCCL) and
the torch restatements, then prints MULTIGPU_OK on rank 0."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from ccbench_b200 import Communicator  # noqa: E402
from ccbench_b200.ops import codecs as C  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=dev)
    want_nvls = os.environ.get("CCB_TEST_NVLS", "1") == "1"
    comm = Communicator.from_torch_distributed(arena_bytes=512 << 20, nvls=want_nvls)
    if rank == 0:
        print("nvls mapping:", comm.has_nvls, flush=True)
    import traceback
    try:
        _body(comm, rank, world, dev)
    except Exception:
        print(f"[rank {rank}] FAILED\n" + traceback.format_exc(), flush=True)
        os._exit(1)
    dist.barrier()
    comm.close()
    if rank == 0:
        print("MULTIGPU_OK", flush=True)
    dist.destroy_process_group()


def _body(comm, rank, world, dev):

    def gather_inputs(x):
        xs = [torch.empty_like(x) for _ in range(world)]
        dist.all_gather(xs, x)
        return [t.cpu() for t in xs]

    for dtype in (torch.float32, torch.bfloat16):
        for count in (1000, 1 << 20, (1 << 22) + 77):
            g = torch.Generator(device=dev).manual_seed(rank * 1000 + count)
            x = (torch.randn(count, generator=g, device=dev) * (rank + 1)).to(dtype)
            xs = gather_inputs(x)
            exact = sum(t.double() for t in xs).float()
            for codec in ("int8", "fp8", "none"):
                for algo in ("twoshot", "oneshot", "ring", "tree"):
                    y = torch.empty_like(x)
                    for _ in range(3):
                        comm.all_reduce(x, y, codec=codec, algo=algo)
                    torch.cuda.synchronize()
                    rc, words = comm.status()
                    assert rc == 0, words
                    want = C.simulate_all_reduce(xs, codec, algo, dtype)
                    got = y.float().cpu()
                    scale = want.abs().max().item()
                    step = {"int8": 1 / 127, "fp8": 1 / 8, "none": 2 ** -7 if dtype != torch.float32 else 1e-6}[codec]
                    ulp = 0.0 if dtype == torch.float32 else 2.0 ** -7
                    d = (got - want).abs()
                    # a rounding flip at one hop (fp32 summation order, FMA) can be carried and
                    # widened by the requantisations of the later hops
                    hops = {"ring": world, "tree": 4, "twoshot": 2, "oneshot": 1}[algo]
                    assert d.max().item() <= (hops * 1.01 * step + ulp) * scale, (dtype, count, codec, algo, d.max().item())
                    assert (d > 1e-5 * scale).float().mean().item() < 0.02, (dtype, count, codec, algo)
                    # all ranks bit-identical
                    ys = gather_inputs(y)
                    assert all(torch.equal(ys[0], t) for t in ys), (codec, algo)
            if comm.has_nvls:
                y = torch.empty_like(x)
                for _ in range(3):
                    comm.all_reduce(x, y, codec="none", algo="nvls")
                torch.cuda.synchronize()
                assert comm.status()[0] == 0
                tol = 1e-5 if dtype == torch.float32 else 2e-2
                rel = ((y.float().cpu() - exact).norm() / exact.norm()).item()
                assert rel < tol, ("nvls", dtype, count, rel)

    # reduce_scatter / all_gather / broadcast / all_to_all
    per = 100003
    x = torch.randn(per * world, device=dev) * (rank + 1)
    xs = gather_inputs(x)
    out = torch.empty(per, device=dev)
    comm.reduce_scatter(x, out, codec="int8")
    torch.cuda.synchronize()
    ex = sum(t[rank * per:(rank + 1) * per].double() for t in xs).float()
    assert ((out.cpu() - ex).norm() / ex.norm()).item() < 0.03
    ag = torch.empty(per * world * world, device=dev)
    comm.all_gather(x, ag, codec="fp8")
    torch.cuda.synchronize()
    want = torch.cat([C.roundtrip(t, "fp8") for t in xs])
    assert torch.equal(ag.cpu(), want)
    b = torch.empty_like(x)
    for root in range(world):
        comm.broadcast(x, b, root=root, codec="int8")
        torch.cuda.synchronize()
        wantb = C.roundtrip(xs[root], "int8")
        if not torch.equal(b.cpu(), wantb):
            bad = (b.cpu() != wantb).nonzero().flatten()
            raise AssertionError(f"broadcast root={root} rank={rank}: {bad.numel()} of {wantb.numel()} differ, first at "
                                 f"{bad[:8].tolist()} got {b.cpu()[bad[:4]].tolist()} want {wantb[bad[:4]].tolist()} "
                                 f"last {bad[-3:].tolist()}")
    a2a = torch.empty_like(x)
    comm.all_to_all(x, a2a, codec="none")
    torch.cuda.synchronize()
    want = torch.cat([t[rank * per:(rank + 1) * per] for t in xs])
    assert torch.equal(a2a.cpu(), want)
    red = torch.zeros_like(x)
    for _ in range(3):
        comm.reduce(x, red, root=world - 1, codec="none")
    torch.cuda.synchronize()
    if rank == world - 1:
        ex = sum(t.double() for t in xs).float()
        assert torch.allclose(red.cpu(), ex, rtol=1e-5, atol=1e-5)
    assert comm.status()[0] == 0
    if os.environ.get("CCB_TEST_SECTIONS", "all") != "all":
        return
    _pipelined_and_plain_launches(comm, rank, world, dev, gather_inputs)
    _sz_and_moe(comm, rank, world, dev, gather_inputs)
    _point_to_point(comm, rank, world, dev)
    _overlapping_calls(comm, rank, world, dev, gather_inputs)


def _pipelined_and_plain_launches(comm, rank, world, dev, gather_inputs):
    """The pipelined two-shot kernel over real peers (with and without the multicast second
    phase), and small grids launched without the cooperative attribute."""
    count = (1 << 23) + 4097
    g = torch.Generator(device=dev).manual_seed(77 + rank)
    x = (torch.randn(count, generator=g, device=dev) * (rank + 1)).to(torch.bfloat16)
    xs = gather_inputs(x)
    exact = sum(t.double() for t in xs).float()
    results = {}
    for name, mode, mc in (("plain", 0, False), ("pipe", 2, False), ("pipe_mc", 2, True)):
        if mc and not comm.has_nvls:
            continue
        comm.set_pipeline(mode, multicast=mc)
        comm.set_waves(4 if mode else 0)
        y = torch.empty_like(x)
        for _ in range(3):
            comm.all_reduce(x, y, codec="int8", algo="twoshot")
        torch.cuda.synchronize()
        assert comm.status()[0] == 0, (name, comm.status())
        results[name] = y.float().cpu()
        rel = ((results[name] - exact).norm() / exact.norm()).item()
        assert rel < 0.03, (name, rel)
        ys = gather_inputs(y)
        assert all(torch.equal(ys[0], t) for t in ys), name
    scale = results["plain"].abs().max().item()
    for name in results:
        d = (results[name] - results["plain"]).abs()
        assert (d > 1e-5 * scale).float().mean().item() < 2e-3, name
    # uncompressed sum in place on symmetric (arena-backed) tensors, reduced inside the switch
    if comm.has_nvls:
        for dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 2e-2)):
            n_el = (1 << 20) + 8
            src = (torch.randn(n_el, generator=g, device=dev) * (rank + 1)).to(dtype)
            want = sum(t.double() for t in gather_inputs(src)).float()
            a = comm.symmetric_empty(n_el, dtype)
            b = comm.symmetric_empty(n_el, dtype)
            a.copy_(src)
            comm.all_reduce(a, b, codec="none", algo="nvls")      # out of place, both in the arena
            torch.cuda.synchronize()
            assert ((b.float().cpu() - want).norm() / want.norm()).item() < tol, ("symm", dtype)
            assert torch.equal(a, src)
            comm.all_reduce(a, codec="none", algo="nvls")         # in place
            torch.cuda.synchronize()
            assert comm.status()[0] == 0
            assert ((a.float().cpu() - want).norm() / want.norm()).item() < tol, ("symm in place", dtype)
            # ordinary collectives still work with the smaller staging
            y2 = torch.empty_like(src)
            comm.all_reduce(src, y2, codec="int8", algo="twoshot")
            torch.cuda.synchronize()
            assert ((y2.float().cpu() - want).norm() / want.norm()).item() < 0.03
            comm.symmetric_free_all()
    # reduce_scatter through the pipelined kernel
    per = 1 << 21
    xr = torch.randn(per * world, device=dev) * (rank + 1)
    xrs = gather_inputs(xr)
    out = torch.empty(per, device=dev)
    comm.set_pipeline(2)
    comm.set_waves(4)
    comm.reduce_scatter(xr, out, codec="int8")
    torch.cuda.synchronize()
    ex = sum(t[rank * per:(rank + 1) * per].double() for t in xrs).float()
    assert ((out.cpu() - ex).norm() / ex.norm()).item() < 0.03
    comm.set_pipeline(1)
    comm.set_waves(0)
    # few CTAs, plain (non-cooperative) launches: what the overlap benchmark uses
    comm.set_max_ctas(8)
    comm.set_noncooperative(8)
    for algo in ("twoshot", "ring"):
        y = torch.empty_like(x)
        for _ in range(3):
            comm.all_reduce(x, y, codec="int8", algo=algo)
        torch.cuda.synchronize()
        assert comm.status()[0] == 0
        assert ((y.float().cpu() - exact).norm() / exact.norm()).item() < 0.06, algo
    comm.reduce_scatter(xr, out, codec="int8")
    torch.cuda.synchronize()
    assert ((out.cpu() - ex).norm() / ex.norm()).item() < 0.03
    comm.set_max_ctas(0)
    comm.set_noncooperative(0)
    assert comm.status()[0] == 0


def _overlapping_calls(comm, rank, world, dev, gather_inputs):
    """Consecutive pipelined calls that may overlap tail and head: different inputs and
    alternating outputs, every result equal to what the same call gives alone, and a kernel
    put on the stream afterwards sees all of them."""
    count = (1 << 22) + 4097
    xs = [(torch.randn(count, generator=torch.Generator(device=dev).manual_seed(300 + 7 * k + rank), device=dev) * (k + 1)).to(torch.bfloat16)
          for k in range(3)]
    alone = []
    comm.set_pipeline(2)
    for x in xs:
        y = torch.empty_like(x)
        comm.all_reduce(x, y, codec="int8", algo="twoshot")
        alone.append(y)
    torch.cuda.synchronize()
    comm.set_call_overlap(True)
    outs = [torch.zeros_like(x) for x in xs]
    for rep in range(3):
        for k in range(3):
            comm.all_reduce(xs[k], outs[k], codec="int8", algo="twoshot")
    total = sum(o.float().sum() for o in outs)          # ordinary kernels, ordered after every call
    torch.cuda.synchronize()
    comm.set_call_overlap(False)
    comm.set_pipeline(1)
    assert comm.status()[0] == 0, comm.status()
    for k in range(3):
        assert torch.equal(outs[k], alone[k]), ("overlapping calls", k)
    assert torch.isfinite(total)


def _point_to_point(comm, rank, world, dev):
    """Sends and receives over the arena mailboxes: a ring shift in one grouped launch, odd
    byte counts and unaligned starts, a message of many rounds, and two messages to the same
    peer in one call (which the runtime puts into consecutive launches)."""
    nxt, prv = (rank + 1) % world, (rank - 1) % world

    def payload(r, n, salt):
        return (torch.arange(n, dtype=torch.int64) * (2 * r + 3) + salt).to(torch.uint8)

    for n, salt in ((1, 1), (4099, 2), (1 << 20, 3), ((48 << 20) + 7, 4)):
        mine = payload(rank, n + 3, salt).to(dev)
        got = torch.zeros(n + 5, dtype=torch.uint8, device=dev)
        comm.p2p([("send", mine[3:], nxt), ("recv", got[5:], prv)])   # starts off a 16-byte boundary
        torch.cuda.synchronize()
        assert comm.status()[0] == 0, comm.status()
        assert torch.equal(got[5:].cpu(), payload(prv, n + 3, salt)[3:]), ("p2p ring", n)
        assert int(got[:5].sum()) == 0
    a, b = payload(rank, 70001, 5).to(dev), payload(rank, 333, 6).to(dev)
    ra, rb = torch.zeros(70001, dtype=torch.uint8, device=dev), torch.zeros(333, dtype=torch.uint8, device=dev)
    comm.p2p([("send", a, nxt), ("send", b, nxt), ("recv", ra, prv), ("recv", rb, prv)])
    torch.cuda.synchronize()
    assert torch.equal(ra.cpu(), payload(prv, 70001, 5)) and torch.equal(rb.cpu(), payload(prv, 333, 6))
    # everyone to everyone in one launch (float payload)
    x = torch.full((world, 5000), float(rank), device=dev) + torch.arange(world, device=dev)[:, None] * 0.5
    y = torch.zeros_like(x)
    ops = []
    for p in range(world):
        if p != rank:
            ops += [("send", x[p], p), ("recv", y[p], p)]
    comm.p2p(ops)
    torch.cuda.synchronize()
    for p in range(world):
        if p != rank:
            assert torch.equal(y[p].cpu(), torch.full((5000,), float(p)) + rank * 0.5), ("p2p all pairs", p)
    assert comm.status()[0] == 0


def _sz_and_moe(comm, rank, world, dev, gather_inputs):
    """Error-bounded AllGather / Broadcast and MoE dispatch + combine over real peers."""
    from ccbench_b200.models.workloads import moe_routing, smooth_field
    from ccbench_b200.ops import sz
    from ccbench_b200.parallel import moe

    n = 96
    fld = smooth_field(n, seed=rank, device=dev)
    flds = gather_inputs(fld)
    eb = 1e-3 * max((f.max() - f.min()).item() for f in flds)
    eb32 = float(torch.tensor(eb, dtype=torch.float32))
    recv = torch.zeros((world, n, n, n), device=dev)
    for it in range(3):
        sz.all_gather(comm, fld, recv, eb)
        if rank == 0 and it == 0:
            print("sz launch path:", sz.launch_path(), "(1 = cluster + cooperative, 2 = cluster alone)", flush=True)
    torch.cuda.synchronize()
    assert comm.status()[0] == 0
    for q in range(world):
        assert (recv[q].cpu() - flds[q]).abs().max().item() <= eb32, ("sz all_gather bound", q)
        buf, _ = sz.compress(flds[q].to(dev), eb)
        assert torch.equal(recv[q], sz.decompress(buf, fld.shape, eb)), ("sz all_gather vs local codec", q)
    out = torch.zeros_like(fld)
    for root in (0, world - 1):
        for _ in range(2):
            sz.broadcast(comm, fld, out, eb, root=root)
        torch.cuda.synchronize()
        assert comm.status()[0] == 0
        assert (out.cpu() - flds[root]).abs().max().item() <= eb32, ("sz broadcast bound", root)

    T, H, dt = 300, 1024, torch.bfloat16
    x = torch.randn(T, H, generator=torch.Generator().manual_seed(rank)).to(dt).to(dev)
    ids, gates = moe_routing(T, world, 2, seed=rank)
    rt = moe.plan_route(ids, gates, world)
    counts = [None] * world
    dist.all_gather_object(counts, rt.send_counts.tolist())
    route = moe.Route(rt.perm.to(dev), rt.dest_rank.to(dev), rt.pos.to(dev), rt.gate.to(dev), rt.send_counts, rt.topk)
    rows_in = sum(counts[s][rank] for s in range(world))
    for codec in ("fp8", "none"):
        recv = torch.zeros(max(rows_in, 1), H, dtype=dt, device=dev)
        for _ in range(2):
            moe.dispatch(comm, x, recv, route, counts, codec=codec)
        torch.cuda.synchronize()
        assert comm.status()[0] == 0
        xs = gather_inputs(x)
        perms = [None] * world
        dist.all_gather_object(perms, rt.perm.tolist())
        want = []
        for s in range(world):
            start = sum(counts[s][:rank])
            rows = torch.tensor(perms[s][start:start + counts[s][rank]], dtype=torch.long)
            want.append(C.roundtrip(xs[s][rows].float(), codec, dt).to(dt).reshape(-1, H))
        want = torch.cat(want)
        assert torch.equal(recv[:rows_in].cpu(), want), ("moe dispatch", codec)
        # identity experts: combine returns every token gate-weighted (gates sum to 1)
        out = torch.zeros(T, H, dtype=dt, device=dev)
        moe.combine(comm, recv, out, route, counts, codec=codec)
        torch.cuda.synchronize()
        assert comm.status()[0] == 0
        tol = {"fp8": 0.15, "none": 0.02}[codec]
        rel = ((out.float() - x.float()).norm() / x.float().norm()).item()
        assert rel < tol, ("moe combine", codec, rel)


if __name__ == "__main__":
    main()
