"""ccb_all_reduce_noalloc, called through its exported C symbol, against the ordinary
entry point (a local communicator's all_reduce).

The no-alloc entry point is for callers that may not allocate GPU memory where they
need the collective (a plugin inside another program's latency-critical loop, a
callback that runs while a caching allocator owns all free memory): its staging lives
in a static device array inside libccb.so. It runs the same kernel as the ordinary
entry point, so the results must agree; the check uses the tolerance of the other GPU
tests. Two calls in a row exercise the reuse of the shared array (its flags are
ordered by a call counter, not cleared). This file sorts last on purpose, so that a
run stopping at the first failure has already run every other test."""
import ctypes

import pytest
import torch

from ccbench_b200 import Communicator, constants as K
from ccbench_b200._lib import lib

pytestmark = pytest.mark.gpu

_DT = {torch.float32: K.F32, torch.bfloat16: K.BF16, torch.float16: K.F16}


def _noalloc(xs, outs, codec):
    L = lib()
    L.ccb_all_reduce_noalloc.argtypes = [ctypes.POINTER(ctypes.c_void_p), ctypes.POINTER(ctypes.c_void_p), ctypes.c_int,
                                         ctypes.c_uint64, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    L.ccb_all_reduce_noalloc.restype = ctypes.c_int
    n = len(xs)
    sp = (ctypes.c_void_p * n)(*[x.data_ptr() for x in xs])
    rp = (ctypes.c_void_p * n)(*[o.data_ptr() for o in outs])
    return L.ccb_all_reduce_noalloc(sp, rp, n, xs[0].numel(), _DT[xs[0].dtype], K.CODECS[codec],
                                    ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("codec", ["int8", "fp8", "none"])
@pytest.mark.parametrize("n,count", [(4, 20000), (2, 4097), (3, 512), (1, 3000)])
def test_matches_the_ordinary_entry_point_twice(dtype, codec, n, count):
    comm = Communicator.local(n, arena_bytes=8 << 20)
    try:
        for call in range(2):  # two calls in a row share the static array
            g = torch.Generator().manual_seed(100 * call + n)
            xs = [(torch.randn(count, generator=g) * (r + 1)).to(dtype).cuda() for r in range(n)]
            want = [torch.empty_like(x) for x in xs]
            comm.all_reduce(xs, want, codec=codec, algo="twoshot")
            got = [torch.full_like(x, float("nan")) for x in xs]
            rc = _noalloc(xs, got, codec)
            assert rc == 0, lib().ccb_last_error()
            torch.cuda.synchronize()
            scale = want[0].float().abs().max().item() + 1e-30
            step = {"int8": 1 / 127, "fp8": 1 / 8, "none": 2 ** -7 if dtype != torch.float32 else 1e-6}[codec]
            ulp = 0.0 if dtype == torch.float32 else 2.0 ** -7
            words = (ctypes.c_uint32 * 8)()
            assert lib().ccb_noalloc_status(words) == 0 and words[0] == 0, "no device-side wait may have given up"
            for r in range(n):
                d = (got[r].float() - want[r].float()).abs().max().item()
                assert d <= (2 * 1.01 * step + ulp) * scale, (call, r, d)
                assert torch.equal(got[r], got[0])
    finally:
        comm.close()


def test_rejects_sizes_beyond_the_built_in_scratch():
    L = lib()
    L.ccb_noalloc_max_count.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int]
    L.ccb_noalloc_max_count.restype = ctypes.c_uint64
    limit = L.ccb_noalloc_max_count(4, K.F32, K.CODEC_NONE)
    assert 0 < limit < (1 << 22)
    xs = [torch.ones(limit + 512, device="cuda") for _ in range(4)]
    outs = [torch.zeros_like(x) for x in xs]
    assert _noalloc(xs, outs, "none") == K.ERR_CAPACITY
    assert b"exceed" in L.ccb_last_error()
    torch.cuda.synchronize()
    assert outs[0].abs().sum().item() == 0  # nothing was launched
    ok = [torch.ones(limit, device="cuda") for _ in range(4)]
    res = [torch.zeros_like(x) for x in ok]
    assert _noalloc(ok, res, "none") == 0
    torch.cuda.synchronize()
    assert res[3].eq(4.0).all()
    assert L.ccb_noalloc_max_count(5, K.F32, K.CODEC_NONE) == 0
