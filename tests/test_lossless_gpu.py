"""The lossless float kernels against the NumPy restatement of the container: the used part
of every slot byte for byte, the round trip bit for bit, decode-add, and the hook library."""
import ctypes
from pathlib import Path

import numpy as np
import pytest
import torch

from ccbench_b200.ops import lossless as LL

pytestmark = pytest.mark.gpu
CODES = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}
LIBS = Path(__file__).resolve().parent.parent / "bin" / "libs"


def _bits(x):
    x = x.cpu()
    return x.view(torch.int32).numpy().view(np.uint32) if x.dtype == torch.float32 else x.view(torch.int16).numpy().view(np.uint16)


def _data(count, dtype, seed=0):
    g = torch.Generator().manual_seed(seed)
    x = (torch.randn(count, generator=g) * 10.0 ** torch.randint(-5, 3, (count,), generator=g)).to(dtype)
    x[::89] = 0.0
    if count > 20:
        x[2], x[5], x[9] = float("inf"), float("nan"), -0.0
    return x


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("count", [1, 100, 512, 2048, 4096, 4097, 70001, 1 << 20])
def test_container_matches_the_restatement_and_round_trips(dtype, count):
    x = _data(count, dtype, seed=count)
    xg = x.cuda()
    comp = LL.encode(xg)
    back = LL.decode(comp, count, dtype)
    torch.cuda.synchronize()
    assert np.array_equal(_bits(back), _bits(x)), "round trip must be bit-exact"
    want = LL.np_encode(_bits(x), CODES[dtype])
    got = comp.cpu().numpy()
    assert got.size == want.size
    assert np.array_equal(got[:32], want[:32]), "header (magic, type, count, used bytes)"
    sb = LL.slot_bytes(CODES[dtype])
    for t in range((count + LL.TILE - 1) // LL.TILE):
        a, b = got[32 + t * sb:32 + (t + 1) * sb], want[32 + t * sb:32 + (t + 1) * sb]
        used = int(b[:4].view(np.uint32)[0])
        assert np.array_equal(a[:used], b[:used]), f"slot {t}"
    assert LL.used_bytes(comp) == LL.used_bytes_np(want)
    # and the restatement decodes what the GPU wrote
    assert np.array_equal(LL.np_decode(got), _bits(x))


def test_decode_add_and_ratio_on_gradient_like_data():
    from ccbench_b200.models.workloads import gradient_like

    x = gradient_like(1 << 22, torch.bfloat16, seed=1, device="cuda")
    comp = LL.encode(x)
    acc = torch.ones_like(x)
    LL.decode(comp, x.numel(), x.dtype, out=acc, accumulate=True)
    torch.cuda.synchronize()
    assert torch.equal(acc, (x.float() + 1).to(torch.bfloat16))
    r = x.numel() * 2 / LL.used_bytes(comp)
    assert 1.15 < r < 2.0, r


def test_hook_library_round_trip_and_reduce():
    path = LIBS / "libdietgpu_wrapper.so"
    assert path.exists(), f"{path} is not built (python -m ccbench_b200.cli build)"
    L = ctypes.CDLL(str(path))
    vp, sz, i = ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int
    L.ncclCompressedChunkBytes.argtypes, L.ncclCompressedChunkBytes.restype = [sz, i], sz
    L.ncclCompress.argtypes = [vp, ctypes.POINTER(vp), sz, i, ctypes.POINTER(sz), ctypes.POINTER(i), sz, i, i, vp]
    L.ncclDecompress.argtypes = [vp, vp, sz, i, sz, i, sz, i, vp]
    L.ncclDecompressReduce.argtypes = [vp, vp, sz, i, sz, i, sz, i, vp]
    L.ncclDecompReduceComp.argtypes = [vp, ctypes.POINTER(vp), sz, i, sz, i, ctypes.POINTER(sz), ctypes.POINTER(i), sz, i, vp]
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    chunks, per, F32, U8 = 3, 5000, 7, 1
    x = torch.randn(chunks * per, generator=torch.Generator().manual_seed(4)).cuda()
    stride = L.ncclCompressedChunkBytes(per, F32)
    assert stride == LL.max_bytes(0, per)
    comp = torch.zeros(stride * chunks, dtype=torch.uint8, device="cuda")
    p, cc, cd = vp(comp.data_ptr()), sz(0), i(-1)
    assert L.ncclCompress(x.data_ptr(), ctypes.byref(p), per, F32, ctypes.byref(cc), ctypes.byref(cd), chunks, 0, 2, stream) == 0
    assert cc.value == stride and cd.value == U8
    out = torch.empty_like(x)
    assert L.ncclDecompress(out.data_ptr(), comp.data_ptr(), per, F32, stride, U8, chunks, 2, stream) == 0
    acc = torch.full_like(x, 2.0)
    assert L.ncclDecompressReduce(acc.data_ptr(), comp.data_ptr(), stride, U8, per, F32, chunks, 2, stream) == 0
    q, rc, rd = vp(None), sz(0), i(-1)
    assert L.ncclDecompReduceComp(comp.data_ptr(), ctypes.byref(q), per, F32, stride, U8, ctypes.byref(rc), ctypes.byref(rd), chunks, 2, stream) == 0
    one = torch.empty(per, device="cuda")
    assert L.ncclDecompress(one.data_ptr(), q, per, F32, rc.value, U8, 1, 2, stream) == 0
    torch.cuda.synchronize()
    assert torch.equal(out, x)
    assert torch.equal(acc, x + 2.0)
    v = x.view(chunks, per)
    assert torch.equal(one, (v[0] + v[1]) + v[2])
