"""The four compression hooks (ncclCompress, ncclDecompress, ncclDecompressReduce,
ncclDecompReduceComp) of the two hook libraries, called through ctypes the way an NCCL fork
with compression support would call them."""
import ctypes
import os
from pathlib import Path

import pytest
import torch

from ccbench_b200.ops import codecs as C

pytestmark = pytest.mark.gpu
LIBS = Path(__file__).resolve().parent.parent / "bin" / "libs"
NCCL_F32, NCCL_F16, NCCL_BF16, NCCL_U8 = 7, 6, 9, 1
DT = {torch.float32: NCCL_F32, torch.float16: NCCL_F16, torch.bfloat16: NCCL_BF16}


def _load(name):
    path = LIBS / name
    assert path.exists(), f"{path} is not built (python -m ccbench_b200.cli build)"
    L = ctypes.CDLL(str(path))
    vp, sz, i = ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int
    L.ncclCompressedChunkBytes.argtypes, L.ncclCompressedChunkBytes.restype = [sz, i], sz
    L.ncclCompress.argtypes = [vp, ctypes.POINTER(vp), sz, i, ctypes.POINTER(sz), ctypes.POINTER(i), sz, i, i, vp]
    L.ncclDecompress.argtypes = [vp, vp, sz, i, sz, i, sz, i, vp]
    L.ncclDecompressReduce.argtypes = [vp, vp, sz, i, sz, i, sz, i, vp]
    L.ncclDecompReduceComp.argtypes = [vp, ctypes.POINTER(vp), sz, i, sz, i, ctypes.POINTER(sz), ctypes.POINTER(i), sz, i, vp]
    return L


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _compress(L, x, chunks):
    per = x.numel() // chunks
    stride = L.ncclCompressedChunkBytes(per, DT[x.dtype])
    comp = torch.zeros(stride * chunks, dtype=torch.uint8, device="cuda")
    p, cc, cd = ctypes.c_void_p(comp.data_ptr()), ctypes.c_size_t(0), ctypes.c_int(-1)
    assert L.ncclCompress(x.data_ptr(), ctypes.byref(p), per, DT[x.dtype], ctypes.byref(cc), ctypes.byref(cd), chunks, 0, 2, _stream()) == 0
    assert cc.value == stride and cd.value == NCCL_U8 and p.value == comp.data_ptr()
    return comp, stride, per


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("bits", [4, 8])
def test_sdp4bit_layout_and_round_trip(dtype, bits, monkeypatch):
    monkeypatch.setenv("SDP4BIT_BITS", str(bits))
    monkeypatch.setenv("SDP4BIT_GROUP", "256")
    import subprocess
    import sys

    # the library caches its environment on first use: run the body in a fresh process
    code = f"""
import ctypes, torch, sys
sys.path.insert(0, {str(Path(__file__).resolve().parent.parent)!r})
sys.path.insert(0, {str(Path(__file__).resolve().parent)!r})
import test_hooks_gpu as T
L = T._load("libsdp4bit.so")
chunks, per, bits, group = 3, 5000, {bits}, 256
x = (torch.randn(chunks * per, generator=torch.Generator().manual_seed(1)) * 2).to({dtype}).cuda()
comp, stride, per = T._compress(L, x, chunks)
groups = (per + group - 1) // group
assert stride == (16 + 4 * groups + (per if bits == 8 else (per + 1) // 2) + 15) // 16 * 16
head = comp[:16].view(torch.int32).tolist()
assert head[:3] == [groups, bits, group], head
out = torch.empty_like(x)
assert L.ncclDecompress(out.data_ptr(), comp.data_ptr(), per, T.DT[x.dtype], stride, T.NCCL_U8, chunks, 2, T._stream()) == 0
qmax = 127.0 if bits == 8 else 7.0
xf = x.float().cpu().view(chunks, per)
for c in range(chunks):
    pad = (-per) % group
    xc = torch.cat([xf[c], torch.zeros(pad)]).view(-1, group)
    m = xc.abs().amax(dim=1, keepdim=True)
    inv = torch.where(m > 0, torch.full_like(m, qmax) / m, torch.zeros_like(m))
    want = (torch.round(xc * inv) * (m / torch.full_like(m, qmax))).view(-1)[:per].to({dtype}).float()
    got = out.float().cpu().view(chunks, per)[c]
    assert torch.equal(got, want), (c, (got - want).abs().max())
acc = torch.ones_like(x)
assert L.ncclDecompressReduce(acc.data_ptr(), comp.data_ptr(), stride, T.NCCL_U8, per, T.DT[x.dtype], chunks, 2, T._stream()) == 0
assert torch.allclose(acc.float(), out.float() + 1, atol=7e-2 if x.dtype != torch.float32 else 1e-6)
p, rc, rd = ctypes.c_void_p(None), ctypes.c_size_t(0), ctypes.c_int(-1)
assert L.ncclDecompReduceComp(comp.data_ptr(), ctypes.byref(p), per, T.DT[x.dtype], stride, T.NCCL_U8, ctypes.byref(rc), ctypes.byref(rd), chunks, 2, T._stream()) == 0
one = torch.empty(per, dtype=x.dtype, device="cuda")
assert L.ncclDecompress(one.data_ptr(), p, per, T.DT[x.dtype], rc.value, T.NCCL_U8, 1, 2, T._stream()) == 0
torch.cuda.synchronize()
total = out.float().view(chunks, per).sum(0)
step = total.abs().max().item() / qmax
ulp = 0.0 if x.dtype == torch.float32 else total.abs().max().item() * 2.0 ** -8
assert (one.float() - total).abs().max().item() <= 0.51 * step * 1.3 + ulp + 1e-6
print("HOOKS_OK")
"""
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=dict(os.environ), timeout=300)
    assert "HOOKS_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-3000:]


def test_fused_hook_library_round_trip():
    L = _load("libccb_coccl_hooks.so")
    chunks, per = 4, 4096 + 512
    x = torch.randn(chunks * per, generator=torch.Generator().manual_seed(2)).cuda()
    comp, stride, per = _compress(L, x, chunks)
    out = torch.empty_like(x)
    assert L.ncclDecompress(out.data_ptr(), comp.data_ptr(), per, NCCL_F32, stride, NCCL_U8, chunks, 2, _stream()) == 0
    want = torch.cat([C.roundtrip(x.cpu()[c * per:(c + 1) * per], "int8") for c in range(chunks)])
    assert torch.equal(out.cpu(), want)
    acc = torch.zeros_like(x)
    assert L.ncclDecompressReduce(acc.data_ptr(), comp.data_ptr(), stride, NCCL_U8, per, NCCL_F32, chunks, 2, _stream()) == 0
    assert torch.equal(acc.cpu(), want)
    p, rc, rd = ctypes.c_void_p(None), ctypes.c_size_t(0), ctypes.c_int(-1)
    assert L.ncclDecompReduceComp(comp.data_ptr(), ctypes.byref(p), per, NCCL_F32, stride, NCCL_U8, ctypes.byref(rc), ctypes.byref(rd), chunks, 2, _stream()) == 0
    one = torch.empty(per, device="cuda")
    assert L.ncclDecompress(one.data_ptr(), p, per, NCCL_F32, rc.value, NCCL_U8, 1, 2, _stream()) == 0
    torch.cuda.synchronize()
    total = want.view(chunks, per).sum(0)
    assert (one.cpu() - total).abs().max().item() <= 0.51 / 127 * total.abs().max().item() * 1.05


def test_all_chunks_of_a_hook_call_are_one_launch():
    """An 8-chunk ring step is one kernel per hook, not one per chunk, also with a chunk
    size that is not a multiple of the 512-element wire unit."""
    L = _load("libccb_coccl_hooks.so")
    core = ctypes.CDLL(str(LIBS / "libccb.so"))   # the copy the hook library is linked against
    core.ccb_launch_count.restype = ctypes.c_uint64
    launch_count = core.ccb_launch_count
    chunks, per = 8, 3000
    x = torch.randn(chunks * per, generator=torch.Generator().manual_seed(5)).to(torch.bfloat16).cuda()
    torch.cuda.synchronize()
    n0 = launch_count()
    comp, stride, per = _compress(L, x, chunks)
    assert launch_count() - n0 == 1
    out = torch.empty_like(x)
    assert L.ncclDecompress(out.data_ptr(), comp.data_ptr(), per, NCCL_BF16, stride, NCCL_U8, chunks, 2, _stream()) == 0
    acc = torch.ones_like(x)
    assert L.ncclDecompressReduce(acc.data_ptr(), comp.data_ptr(), stride, NCCL_U8, per, NCCL_BF16, chunks, 2, _stream()) == 0
    assert launch_count() - n0 == 3
    torch.cuda.synchronize()
    want = torch.cat([C.roundtrip(x.cpu()[c * per:(c + 1) * per], "int8") for c in range(chunks)])
    assert torch.equal(out.cpu(), want.float().to(torch.bfloat16))
    # decode and add contract into one fused multiply-add: equal up to one rounding of the 16-bit result
    assert (acc.cpu().float() - (want.float() + 1)).abs().max().item() <= 2.0 ** -7 * (want.abs().max().item() + 1)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_user_template_of_the_four_hooks_with_its_example_codec(dtype):
    """userconfig/wrapper_code_examples/compression/coccl_wrapper_template.cu as shipped (fp16
    values relative to a per-group absmax): round trip, decode + add, and the one-pass sum of
    all chunks re-encoded, every hook one launch for all chunks; odd chunk length."""
    L = _load("libcoccl_wrapper_template.so")
    chunks, per = 5, 4096 + 37
    x = torch.randn(chunks * per, generator=torch.Generator().manual_seed(5)).to(dtype).cuda()
    comp, stride, per = _compress(L, x, chunks)
    assert stride < per * 4 and stride % 16 == 0
    out = torch.empty_like(x)
    assert L.ncclDecompress(out.data_ptr(), comp.data_ptr(), per, DT[dtype], stride, NCCL_U8, chunks, 2, _stream()) == 0
    tol = 2e-3 if dtype == torch.float32 else 1.2e-2
    ref = x.float()
    assert ((out.float() - ref).abs() <= tol * ref.abs().view(chunks, per).amax(1, keepdim=True).expand(chunks, per).reshape(-1) + 1e-6).all()
    acc = torch.ones_like(x)
    assert L.ncclDecompressReduce(acc.data_ptr(), comp.data_ptr(), stride, NCCL_U8, per, DT[dtype], chunks, 2, _stream()) == 0
    assert torch.allclose(acc.float(), out.float() + 1, rtol=1e-2, atol=1e-2)
    p, rc, rd = ctypes.c_void_p(None), ctypes.c_size_t(0), ctypes.c_int(-1)
    assert L.ncclDecompReduceComp(comp.data_ptr(), ctypes.byref(p), per, DT[dtype], stride, NCCL_U8, ctypes.byref(rc), ctypes.byref(rd),
                                  chunks, 2, _stream()) == 0
    one = torch.empty(per, dtype=dtype, device="cuda")
    assert rc.value == stride and L.ncclDecompress(one.data_ptr(), p, per, DT[dtype], rc.value, NCCL_U8, 1, 2, _stream()) == 0
    torch.cuda.synchronize()
    total = out.float().view(chunks, per).sum(0)
    assert (one.float() - total).abs().max().item() <= 1.5e-2 * total.abs().max().item()
