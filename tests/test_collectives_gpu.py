"""Numerics of the fused collective kernels against plain PyTorch fp32 restatements.

All ranks are played on ONE GPU by a single cooperative launch
(`Communicator.local`), so the full flag protocol runs on a one-GPU box."""
import pytest
import torch

from ccbench_b200 import Communicator
from ccbench_b200.ops import codecs as C

pytestmark = pytest.mark.gpu

DT = {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16}


@pytest.fixture(scope="module")
def comms():
    cache = {}

    def get(n):
        if n not in cache:
            cache[n] = Communicator.local(n, arena_bytes=96 << 20)
        return cache[n]

    yield get
    for c in cache.values():
        c.close()


def _inputs(n, count, dtype, seed=0):
    g = torch.Generator().manual_seed(seed)
    xs = [(torch.randn(count, generator=g) * (1 + r)).to(dtype) for r in range(n)]
    return xs, [x.cuda() for x in xs]


def _close(got, want, exact_ref, codec, dtype, hops=2):
    """got vs the simulated algorithm: equal up to fp32 summation-order noise, which can
    flip the rounding of an occasional code; and bounded against the exact sum."""
    got = got.float().cpu()
    diff = (got - want).abs()
    scale = want.abs().max().item() + 1e-30
    step = {"int8": 1 / 127, "int8_g256": 1 / 127, "int4": 1 / 7, "fp8": 1 / 8, "none": 2 ** -7 if dtype != torch.float32 else 1e-6}[codec]
    ulp = 0.0 if dtype == torch.float32 else 2.0 ** -7  # one rounding flip of the 16-bit output
    assert diff.max().item() <= (hops * 1.01 * step + ulp) * scale, f"max diff {diff.max().item()} vs step {step * scale}"
    frac = (diff > 1e-5 * scale).float().mean().item()
    assert frac < 0.02, f"{frac:.4f} of elements differ from the restated algorithm"
    rel = ((got - exact_ref).norm() / (exact_ref.norm() + 1e-30)).item()
    lim = {"int8": 0.03, "int8_g256": 0.04, "int4": 0.45, "fp8": 0.08, "none": 0.01 if dtype != torch.float32 else 1e-5}[codec]
    assert rel < lim, f"relative L2 error {rel}"


@pytest.mark.parametrize("algo", ["twoshot", "oneshot", "ring", "tree"])
@pytest.mark.parametrize("codec", ["int8", "fp8", "none", "int8_g256", "int4"])
@pytest.mark.parametrize("dt", ["f32", "bf16"])
@pytest.mark.parametrize("n,count", [(2, 4096), (4, 70001), (8, 1 << 18), (3, 1000), (1, 5000)])
def test_all_reduce(comms, algo, codec, dt, n, count):
    dtype = DT[dt]
    comm = comms(n)
    xs, xg = _inputs(n, count, dtype)
    out = [torch.empty_like(x) for x in xg]
    comm.all_reduce(xg, out, codec=codec, algo=algo)
    torch.cuda.synchronize()
    assert comm.status()[0] == 0
    want = C.simulate_all_reduce(xs, codec, algo, dtype)
    exact = sum(x.double() for x in xs).float()
    hops = {"ring": max(n, 2), "tree": 4, "twoshot": 2, "oneshot": 2}[algo]
    for r in range(n):
        _close(out[r], want, exact, codec, dtype, hops)
        assert torch.equal(out[r], out[0]), "ranks must hold bit-identical results"


def test_all_reduce_f16_inplace_and_repeat(comms):
    n, count = 4, 33000
    comm = comms(n)
    for it in range(5):  # alternates the staging halves and reuses flags
        xs, xg = _inputs(n, count, torch.float16, seed=it)
        comm.all_reduce(xg, codec="int8", algo="twoshot")
        torch.cuda.synchronize()
        want = C.simulate_all_reduce(xs, "int8", "twoshot", torch.float16)
        exact = sum(x.double() for x in xs).float()
        _close(xg[0], want, exact, "int8", torch.float16)


@pytest.mark.parametrize("op", ["sum", "max", "min", "prod"])
def test_all_reduce_ops_uncompressed(comms, op):
    n, count = 4, 9000
    comm = comms(n)
    g = torch.Generator().manual_seed(1)
    xs = [torch.rand(count, generator=g) + 0.5 for _ in range(n)]
    xg = [x.cuda() for x in xs]
    out = [torch.empty_like(x) for x in xg]
    comm.all_reduce(xg, out, op=op, codec="none", algo="twoshot")
    torch.cuda.synchronize()
    st = torch.stack(xs)
    want = {"sum": st.sum(0), "max": st.max(0).values, "min": st.min(0).values, "prod": st.prod(0)}[op]
    assert torch.allclose(out[2].cpu(), want, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("codec", ["int8", "fp8", "none"])
@pytest.mark.parametrize("n,per", [(2, 512), (4, 10007), (8, 40000)])
def test_reduce_scatter(comms, codec, n, per):
    comm = comms(n)
    xs, xg = _inputs(n, per * n, torch.float32)
    out = [torch.empty(per, device="cuda") for _ in range(n)]
    comm.reduce_scatter(xg, out, codec=codec)
    torch.cuda.synchronize()
    for r in range(n):
        acc = xs[r][r * per:(r + 1) * per].clone()
        for q in range(n):
            if q != r:
                acc = acc + C.roundtrip(xs[q][r * per:(r + 1) * per], codec)
        exact = sum(x[r * per:(r + 1) * per].double() for x in xs).float()
        _close(out[r], acc, exact, codec, torch.float32)


@pytest.mark.parametrize("codec", ["int8", "none"])
def test_reduce_to_root(comms, codec):
    n, count, root = 4, 12345, 2
    comm = comms(n)
    xs, xg = _inputs(n, count, torch.float32)
    out = [torch.zeros(count, device="cuda") for _ in range(n)]
    for _ in range(3):  # rooted calls rely on the end-of-call handshake
        comm.reduce(xg, out, root=root, codec=codec)
    torch.cuda.synchronize()
    acc = xs[root].clone()
    for q in range(n):
        if q != root:
            acc = acc + C.roundtrip(xs[q], codec)
    _close(out[root], acc, sum(x.double() for x in xs).float(), codec, torch.float32)
    assert out[(root + 1) % n].abs().sum().item() == 0


@pytest.mark.parametrize("codec", ["int8", "fp8", "none"])
@pytest.mark.parametrize("dt", ["f32", "bf16"])
def test_all_gather_and_broadcast(comms, codec, dt):
    n, per = 4, 20011
    dtype = DT[dt]
    comm = comms(n)
    xs, xg = _inputs(n, per, dtype)
    out = [torch.empty(per * n, device="cuda", dtype=dtype) for _ in range(n)]
    comm.all_gather(xg, out, codec=codec)
    torch.cuda.synchronize()
    want = torch.cat([C.roundtrip(x, codec, dtype).to(dtype) for x in xs])
    for r in range(n):
        assert torch.equal(out[r].cpu(), want)
    outb = [torch.zeros(per, device="cuda", dtype=dtype) for _ in range(n)]
    for _ in range(3):
        comm.broadcast(xg, outb, root=1, codec=codec)
    torch.cuda.synchronize()
    wb = C.roundtrip(xs[1], codec, dtype).to(dtype)
    for r in range(n):
        assert torch.equal(outb[r].cpu(), wb)


@pytest.mark.parametrize("codec", ["fp8", "int8", "none"])
def test_all_to_all(comms, codec):
    n, per = 8, 5000
    comm = comms(n)
    xs, xg = _inputs(n, per * n, torch.bfloat16)
    out = [torch.empty(per * n, device="cuda", dtype=torch.bfloat16) for _ in range(n)]
    comm.all_to_all(xg, out, codec=codec)
    torch.cuda.synchronize()
    for d in range(n):
        want = torch.cat([C.roundtrip(xs[s][d * per:(d + 1) * per], codec, torch.bfloat16).to(torch.bfloat16) for s in range(n)])
        assert torch.equal(out[d].cpu(), want)


def test_scatter_gather_and_v(comms):
    n, per, root = 4, 3001, 3
    comm = comms(n)
    xs, xg = _inputs(n, per * n, torch.float32)
    out = [torch.zeros(per, device="cuda") for _ in range(n)]
    comm.scatter(xg, out, root=root)
    torch.cuda.synchronize()
    for r in range(n):
        assert torch.equal(out[r].cpu(), xs[root][r * per:(r + 1) * per])
    small = [x[:per].contiguous() for x in xg]
    big = [torch.zeros(per * n, device="cuda") for _ in range(n)]
    comm.gather(small, big, root=root)
    torch.cuda.synchronize()
    assert torch.equal(big[root].cpu(), torch.cat([x[:per] for x in xs]))
    # allgatherv with uneven counts through the general exchange
    cnts = [100, 2000, 1, 777]
    offs = [0, 100, 2100, 2101]
    counts = [[cnts[s]] * n for s in range(n)]
    so = [[0] * n for _ in range(n)]
    ro = [[offs[s] for s in range(n)] for _ in range(n)]
    outv = [torch.zeros(sum(cnts), device="cuda") for _ in range(n)]
    comm.exchange(xg, outv, counts, so, ro, codec="none")
    torch.cuda.synchronize()
    want = torch.cat([xs[s][:cnts[s]] for s in range(n)])
    for r in range(n):
        assert torch.equal(outv[r].cpu(), want)


def test_error_feedback_reduces_drift(comms):
    """With error feedback the time-average of the compressed sums converges to the
    true sum; without it the bias of repeatedly quantising the same input stays."""
    n, count = 4, 1 << 15
    comm = comms(n)
    xs, xg = _inputs(n, count, torch.float32, seed=3)
    exact = sum(x.double() for x in xs).float()
    for algo in ["twoshot", "ring", "tree", "oneshot"]:
        ef = [torch.zeros(count, device="cuda") for _ in range(n)]
        acc_ef = torch.zeros(count)
        acc_no = torch.zeros(count)
        T = 24
        for _ in range(T):
            o1 = [torch.empty_like(x) for x in xg]
            comm.all_reduce(xg, o1, codec="int8", algo=algo, error_feedback=ef)
            o2 = [torch.empty_like(x) for x in xg]
            comm.all_reduce(xg, o2, codec="int8", algo=algo)
            acc_ef += o1[0].cpu()
            acc_no += o2[0].cpu()
        e_ef = ((acc_ef / T - exact).norm() / exact.norm()).item()
        e_no = ((acc_no / T - exact).norm() / exact.norm()).item()
        assert e_ef < 0.35 * e_no, (algo, e_ef, e_no)


def test_large_message_is_sliced(comms):
    """A message whose staging exceeds half the arena is cut into several launches."""
    n = 2
    comm = comms(n)
    count = 40 << 20  # 160 MiB of fp32 per rank, uncompressed two-shot needs 2x that
    xg = [torch.full((count,), float(r + 1), device="cuda") for r in range(n)]
    comm.all_reduce(xg, codec="none", algo="twoshot")
    torch.cuda.synchronize()
    assert comm.status()[0] == 0
    assert xg[0][::4097].eq(3.0).all() and xg[1][-5:].eq(3.0).all()


def test_wait_timeout_reports_status_and_leaves_the_context_usable():
    """A wait that nothing satisfies runs out and is reported; nothing traps or hangs.
    Rank 1 of a 2-rank communicator never takes part: the launch plays rank 0 only."""
    from ccbench_b200.testing import launch_partial_all_reduce

    comm = Communicator.local(2, arena_bytes=8 << 20)
    comm.set_timeout_ms(200)
    x = torch.ones(4096, device="cuda")
    launch_partial_all_reduce(comm, x, ranks_played=1)
    torch.cuda.synchronize()
    rc, words = comm.status()
    assert rc == 4 and (words[0] & 1) == 1
    with pytest.raises(Exception):
        comm.all_reduce([x, x.clone()], codec="none")
    comm.close()
    # the CUDA context is intact
    assert torch.ones(8, device="cuda").sum().item() == 8
