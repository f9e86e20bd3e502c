"""Error-bounded codec: bound, exact agreement with the NumPy restatement, packed
size, odd shapes (plain-load path), raw tiles, and the fused AllGather / Broadcast with
all ranks played on one GPU."""
import numpy as np
import pytest
import torch

from ccbench_b200 import Communicator
from ccbench_b200.models.workloads import smooth_field
from ccbench_b200.ops import sz

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("shape", [(16, 16, 64), (8, 8, 32), (24, 40, 96), (9, 13, 50), (17, 8, 33)])
@pytest.mark.parametrize("eb", [1e-3, 1e-1])
def test_roundtrip_matches_restatement(shape, eb):
    g = torch.Generator().manual_seed(sum(shape))
    x = torch.randn(shape, generator=g).cumsum(-1).mul_(0.1)
    xg = x.cuda()
    buf, used = sz.compress(xg, eb)
    out = sz.decompress(buf, shape, eb)
    torch.cuda.synchronize()
    recon, nbytes = sz.restate(x.numpy(), eb)
    assert (out.cpu() - x).abs().max().item() <= float(np.float32(eb))  # the bound is the fp32 value of eb
    assert np.array_equal(out.cpu().numpy(), recon)
    assert int(used.item()) == nbytes


def test_smooth_field_ratio_and_bound():
    f = smooth_field(128, seed=1, device="cuda")
    rng = (f.max() - f.min()).item()
    eb = 1e-4 * rng
    buf, used = sz.compress(f, eb)
    out = sz.decompress(buf, f.shape, eb)
    torch.cuda.synchronize()
    assert (out - f).abs().max().item() <= float(np.float32(eb))
    ratio = f.numel() * 4 / int(used.item())
    assert ratio > 2.5, ratio
    mse = ((out - f).double() ** 2).mean().item()
    psnr = 20 * np.log10(rng) - 10 * np.log10(mse)
    assert psnr > 80


def test_non_finite_and_huge_values_are_stored_raw():
    x = torch.randn(8, 8, 64)
    x[0, 0, 0] = float("inf")
    x[3, 2, 40] = 1e30
    xg = x.cuda()
    buf, used = sz.compress(xg, 1e-3)
    out = sz.decompress(buf, x.shape, 1e-3).cpu()
    assert out[0, 0, 0] == float("inf") and out[3, 2, 40] == x[3, 2, 40]
    fin = torch.isfinite(x) & (x.abs() < 1e20)
    assert (out[fin] - x[fin]).abs().max().item() <= float(np.float32(1e-3))


@pytest.mark.parametrize("n", [2, 4])
def test_fused_all_gather_and_broadcast(n):
    shape = (16, 24, 64)
    comm = Communicator.local(n, arena_bytes=64 << 20)
    try:
        g = torch.Generator().manual_seed(n)
        xs = [torch.randn(shape, generator=g).cumsum(-1).mul_(0.05 * (r + 1)) for r in range(n)]
        xg = [x.cuda() for x in xs]
        eb = 1e-3
        recv = [torch.zeros((n,) + shape, device="cuda") for _ in range(n)]
        used = torch.zeros(n, dtype=torch.int64, device="cuda")
        for _ in range(2):
            sz.all_gather(comm, xg, recv, eb, used)
        torch.cuda.synchronize()
        assert comm.status()[0] == 0
        want = np.stack([sz.restate(x.numpy(), eb)[0] for x in xs])
        for r in range(n):
            assert np.array_equal(recv[r].cpu().numpy(), want)
        assert all(int(u) == sz.restate(xs[i].numpy(), eb)[1] for i, u in enumerate(used.tolist()))
        out = [torch.zeros(shape, device="cuda") for _ in range(n)]
        for _ in range(3):
            sz.broadcast(comm, xg, out, eb, root=n - 1)
        torch.cuda.synchronize()
        assert comm.status()[0] == 0
        for r in range(n):
            assert np.array_equal(out[r].cpu().numpy(), want[n - 1])
    finally:
        comm.close()


def test_container_roundtrip_and_file(tmp_path):
    from ccbench_b200.models.workloads import smooth_field

    f = smooth_field(72, seed=5, device="cuda")[:, :60, :68].contiguous()   # ragged tiles on two axes
    eb = 1e-3 * (f.max() - f.min()).item()
    buf, used = sz.compress(f, eb)
    blob = sz.to_container(buf, f.shape, eb)
    assert blob.numel() < f.numel() * 4 / 3
    ngroups = buf.numel() // sz.GROUP_STRIDE
    assert blob.numel() == sz.HEADER_BYTES + 4 * ngroups + int(used.item()) + ngroups * sz.GROUP_HEADER
    back, shape, eb2 = sz.from_container(blob)
    assert tuple(shape) == tuple(f.shape) and eb2 == float(torch.tensor(eb, dtype=torch.float32))
    want = sz.decompress(buf, f.shape, eb)
    assert torch.equal(sz.decompress(back, shape, eb2), want)
    n = sz.save(tmp_path / "field.ccsz", f, eb)
    assert n == blob.numel()
    assert torch.equal(sz.load(tmp_path / "field.ccsz"), want)
    bad = blob.clone()
    bad[0] ^= 0xFF
    with pytest.raises(ValueError):
        sz.from_container(bad)


def test_numpy_codec_reads_gpu_written_bytes_and_the_gpu_reads_numpy_written_bytes():
    """The on-disk container pinned from both sides: what the GPU wrote is decoded by the NumPy
    codec to the very values the GPU decoder produces, and a container written by the NumPy
    encoder is decoded by the GPU kernel to the NumPy decoder's values."""
    g = torch.Generator().manual_seed(11)
    x = torch.randn(20, 19, 70, generator=g).cumsum(-1).mul_(0.05)   # ragged tiles on every axis
    x[3, 4, 5] = 1e30                                                 # forces one raw tile
    eb = 2e-3
    xg = x.cuda()
    buf, _ = sz.compress(xg, eb)
    want = sz.decompress(buf, x.shape, eb).cpu().numpy()
    blob = sz.to_container(buf, x.shape, eb).cpu().numpy()
    assert np.array_equal(sz.decode_cpu(blob), want)
    cpu_blob = sz.encode_cpu(x.numpy(), eb)
    back, shape, eb2 = sz.from_container(torch.from_numpy(cpu_blob).cuda())
    got = sz.decompress(back, shape, eb2).cpu().numpy()
    assert np.array_equal(got, sz.decode_cpu(cpu_blob))
    fin = np.isfinite(x.numpy()) & (np.abs(x.numpy()) < 1e20)
    assert np.abs(got[fin] - x.numpy()[fin]).max() <= float(np.float32(eb))


def test_error_bounded_hook_library():
    """The error-bounded codec behind ncclCompress / ncclDecompress / ncclDecompressReduce /
    ncclDecompReduceComp (the cuZFP wrapper's role): chunk header, bound, reduction."""
    import ctypes
    from pathlib import Path

    path = Path(__file__).resolve().parent.parent / "bin" / "libs" / "libzfp_for_gpu_nvidia.so"
    assert path.exists(), f"{path} is not built (python -m ccbench_b200.cli build)"
    import os

    os.environ["ZFP_PRECISION"] = "10"   # absolute bound 2^-10
    L = ctypes.CDLL(str(path))
    vp, szt, i = ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int
    L.ncclCompressedChunkBytes.argtypes, L.ncclCompressedChunkBytes.restype = [szt, i], szt
    L.ncclCompress.argtypes = [vp, ctypes.POINTER(vp), szt, i, ctypes.POINTER(szt), ctypes.POINTER(i), szt, i, i, vp]
    L.ncclDecompress.argtypes = [vp, vp, szt, i, szt, i, szt, i, vp]
    L.ncclDecompressReduce.argtypes = [vp, vp, szt, i, szt, i, szt, i, vp]
    L.ncclDecompReduceComp.argtypes = [vp, ctypes.POINTER(vp), szt, i, szt, i, ctypes.POINTER(szt), ctypes.POINTER(i), szt, i, vp]
    stream = vp(torch.cuda.current_stream().cuda_stream)
    F32, U8, chunks, per, eb = 7, 1, 3, 8192, 2.0 ** -10
    x = torch.randn(chunks, per, generator=torch.Generator().manual_seed(3)).cumsum(-1).mul_(0.02).cuda()
    stride = L.ncclCompressedChunkBytes(per, F32)
    assert stride > 16
    comp = torch.zeros(stride * chunks, dtype=torch.uint8, device="cuda")
    p, cc, cd = vp(comp.data_ptr()), szt(0), i(-1)
    assert L.ncclCompress(x.data_ptr(), ctypes.byref(p), per, F32, ctypes.byref(cc), ctypes.byref(cd), chunks, 0, 4, stream) == 0
    assert cc.value == stride and cd.value == U8
    out = torch.empty_like(x)
    assert L.ncclDecompress(out.data_ptr(), comp.data_ptr(), per, F32, stride, U8, chunks, 4, stream) == 0
    acc = torch.full_like(x, 1.0)
    assert L.ncclDecompressReduce(acc.data_ptr(), comp.data_ptr(), stride, U8, per, F32, chunks, 2, stream) == 0
    q, rc, rd = vp(None), szt(0), i(-1)
    assert L.ncclDecompReduceComp(comp.data_ptr(), ctypes.byref(q), per, F32, stride, U8, ctypes.byref(rc), ctypes.byref(rd), chunks, 2, stream) == 0
    one = torch.empty(per, device="cuda")
    assert L.ncclDecompress(one.data_ptr(), q, per, F32, rc.value, U8, 1, 2, stream) == 0
    torch.cuda.synchronize()
    assert (out - x).abs().max().item() <= eb
    assert torch.equal(acc, out + 1.0)
    assert (one - out.sum(0)).abs().max().item() <= eb * 1.001
    stream_bytes = comp.view(chunks, stride)[:, :4].contiguous().view(torch.int32).flatten().tolist()
    assert all(0 < b < per * 4 for b in stream_bytes), stream_bytes   # [u32 stream_bytes] and it is smaller than the raw chunk
