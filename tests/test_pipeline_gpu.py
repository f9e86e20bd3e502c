"""The warp-specialised pipelined two-shot kernel against the plain two-shot kernel and the
PyTorch restatement. Both kernels do the same arithmetic in the same order; the compiler
contracts multiply-add pairs differently in the two, so results agree to the last bits of
fp32, and an occasional code lands on the other side of a rounding boundary. The pipelined
kernel is forced on (mode 2) so that small, odd-sized messages exercise partial chunks,
empty waves and every role split."""
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


STEP = {"int8": 1 / 127, "int8_g256": 1 / 127, "int4": 1 / 7, "fp8": 1 / 8, "none": 0.0}


def _same(a, b, codec, what=""):
    """Equal up to fp32 contraction noise: nearly every element within 1e-5 of the scale, the
    rare rounding flip within one quantisation step (plus one ulp of a 16-bit output)."""
    a32, b32 = a.float(), b.float()
    scale = a32.abs().max().item() + 1e-30
    diff = (a32 - b32).abs()
    ulp = 0.0 if a.dtype == torch.float32 else 2.0 ** -7
    assert diff.max().item() <= (1.01 * STEP[codec] + ulp + 1e-5) * scale, f"{what}: max diff {diff.max().item()} at scale {scale}"
    frac = (diff > 1e-5 * scale).float().mean().item()
    assert frac < 2e-3, f"{what}: {frac:.5f} of the elements differ"


def _both(comm, fn):
    """Runs fn() under the plain kernel, then under the pipelined one."""
    comm.set_pipeline(0)
    a = fn()
    comm.set_pipeline(2)
    b = fn()
    comm.set_pipeline(1)
    torch.cuda.synchronize()
    assert comm.status()[0] == 0
    return a, b


@pytest.mark.parametrize("codec", ["int8", "fp8", "none", "int8_g256", "int4"])
@pytest.mark.parametrize("dt", ["f32", "bf16"])
@pytest.mark.parametrize("n,count,waves", [(2, 4096, 1), (4, 70001, 2), (8, 1 << 20, 4), (3, 1000, 3), (8, 3_000_017, 8),
                                           (2, 5_000_000, 0)])
def test_all_reduce_matches_plain_kernel(comms, codec, dt, n, count, waves):
    dtype = DT[dt]
    comm = comms(n)
    comm.set_waves(waves)
    xs, xg = _inputs(n, count, dtype)

    def run():
        out = [torch.empty_like(x) for x in xg]
        comm.all_reduce(xg, out, codec=codec, algo="twoshot")
        torch.cuda.synchronize()
        return out

    plain, piped = _both(comm, run)
    comm.set_waves(0)
    for r in range(n):
        _same(plain[r], piped[r], codec, f"rank {r}")
        assert torch.equal(piped[r], piped[0]), "ranks must hold bit-identical results"
    if count <= 1 << 20:
        want = C.simulate_all_reduce(xs, codec, "twoshot", dtype)
        got = piped[0].float().cpu()
        scale = want.abs().max().item() + 1e-30
        frac = ((got - want).abs() > 1e-5 * scale).float().mean().item()
        assert frac < 0.02, f"{frac:.4f} of elements differ from the restated algorithm"


@pytest.mark.parametrize("link_warps", [1, 15, 30])
def test_role_splits(comms, link_warps):
    n, count = 4, 600_000
    comm = comms(n)
    xs, xg = _inputs(n, count, torch.bfloat16, seed=3)

    def run():
        out = [torch.empty_like(x) for x in xg]
        comm.all_reduce(xg, out, codec="int8", algo="twoshot")
        torch.cuda.synchronize()
        return out

    comm.set_pipeline(0)
    plain = run()
    comm.set_waves(3)
    comm.set_pipeline(2, link_warps=link_warps)
    piped = run()
    comm.set_pipeline(1, link_warps=20)
    comm.set_waves(0)
    assert comm.status()[0] == 0
    for r in range(n):
        _same(plain[r], piped[r], "int8", f"rank {r}")


@pytest.mark.parametrize("codec", ["int8", "fp8", "none"])
@pytest.mark.parametrize("n,per,waves", [(2, 512, 1), (4, 10007, 2), (8, 400_000, 4), (8, 700_001, 8)])
def test_reduce_scatter_matches_plain_kernel(comms, codec, n, per, waves):
    comm = comms(n)
    comm.set_waves(waves)
    xs, xg = _inputs(n, per * n, torch.float32)

    def run():
        out = [torch.empty(per, device="cuda") for _ in range(n)]
        comm.reduce_scatter(xg, out, codec=codec)
        torch.cuda.synchronize()
        return out

    plain, piped = _both(comm, run)
    comm.set_waves(0)
    for r in range(n):
        _same(plain[r], piped[r], codec, f"rank {r}")


def test_error_feedback_and_repeated_calls(comms):
    """Residuals evolve identically under both kernels; repeated calls alternate the staging
    halves and reuse the flag rows."""
    n, count = 4, 300_001
    comm = comms(n)
    comm.set_waves(2)
    xs, xg = _inputs(n, count, torch.bfloat16, seed=5)
    res = {}
    for mode in (0, 2):
        comm.set_pipeline(mode)
        ef = [torch.zeros(count, device="cuda") for _ in range(n)]
        outs = []
        for _ in range(4):
            out = [torch.empty_like(x) for x in xg]
            comm.all_reduce(xg, out, codec="int8", algo="twoshot", error_feedback=ef)
            outs.append(out[1].clone())
        torch.cuda.synchronize()
        res[mode] = (outs, [e.clone() for e in ef])
    comm.set_pipeline(1)
    comm.set_waves(0)
    assert comm.status()[0] == 0
    for a, b in zip(res[0][0], res[2][0]):
        _same(a, b, "int8", "output")
    # a residual is at most half a quantisation step of its group; a flipped code moves it by a step
    for a, b in zip(res[0][1], res[2][1]):
        assert ((a - b).abs() > 1e-3 * a.abs().max()).float().mean().item() < 2e-2


def test_large_message_takes_the_pipelined_kernel_by_default(comms):
    """Default selection: a 32 Mi-element message on two ranks is large enough."""
    n, count = 2, 32 << 20
    comm = comms(n)
    g = torch.Generator(device="cuda").manual_seed(0)
    xg = [torch.randn(count, device="cuda", generator=g).to(torch.bfloat16) for _ in range(n)]
    out = [torch.empty_like(x) for x in xg]
    comm.set_trace(True)
    comm.all_reduce(xg, out, codec="int8", algo="twoshot")
    torch.cuda.synchronize()
    tr = comm.read_trace(4)
    comm.set_trace(False)
    assert comm.status()[0] == 0
    assert int(tr[0, 5]) > 0, "slot 5 (first decoded wave) is written by the pipelined kernel only"
    exact = xg[0].float() + xg[1].float()
    rel = ((out[0].float() - exact).norm() / exact.norm()).item()
    assert rel < 0.03
    assert torch.equal(out[0], out[1])


def test_link_probe_methods_run_and_reject_bad_arguments():
    """The store-method probe on a one-rank communicator (the "peer" is the own arena): vector
    stores and both bulk-copy sizes complete, sizes beyond the data area and unknown methods
    are refused before anything is launched."""
    import ctypes
    import os

    from ccbench_b200._lib import lib
    from ccbench_b200.comm import CcbError, _check

    comm = Communicator.create(0, 1, f"probe{os.getpid()}", arena_bytes=128 << 20)
    try:
        stream = torch.cuda.current_stream().cuda_stream
        for method in (0, 1, 2):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            _check(lib().ccb_link_probe(comm._h, method, 0, 32 << 20, stream))
            e1.record()
            torch.cuda.synchronize()
            assert e0.elapsed_time(e1) > 0 and comm.status()[0] == 0
        for bad in ((3, 0, 1 << 20), (0, 1, 1 << 20), (0, 0, 1 << 40)):
            with pytest.raises(CcbError):
                _check(lib().ccb_link_probe(comm._h, bad[0], bad[1], ctypes.c_uint64(bad[2]), stream))
    finally:
        comm.close()
