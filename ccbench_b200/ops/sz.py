"""Python face of the error-bounded codec (ccb-sz v2) plus a NumPy restatement of its
arithmetic used as the test oracle: the reconstruction q * 2eb and the packed size
must match the kernel's exactly."""
from __future__ import annotations

import ctypes

import numpy as np
import torch

from .._lib import lib
from ..comm import Communicator, _check

TX, TY, TZ = 32, 8, 8


def _decl():
    L = lib()
    c_vp, c_int, c_f = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    L.ccb_sz_capacity.argtypes = [c_int, c_int, c_int]
    L.ccb_sz_capacity.restype = ctypes.c_uint64
    L.ccb_sz_compress.argtypes = [c_vp, c_int, c_int, c_int, c_f, c_vp, c_vp, c_vp]
    L.ccb_sz_decompress.argtypes = [c_vp, c_int, c_int, c_int, c_f, c_vp, c_vp]
    L.ccb_sz_collective.argtypes = [c_vp, ctypes.POINTER(c_vp), ctypes.POINTER(c_vp), c_int, c_int, c_int, c_f, c_int, c_vp, c_vp]
    return L


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def capacity(shape) -> int:
    nz, ny, nx = shape
    return int(_decl().ccb_sz_capacity(nx, ny, nz))


def compress(field: torch.Tensor, eb: float):
    """Returns (buffer uint8 [capacity], used_bytes int). field: fp32 CUDA tensor [nz, ny, nx]."""
    assert field.is_cuda and field.dtype == torch.float32 and field.dim() == 3 and field.is_contiguous()
    nz, ny, nx = field.shape
    buf = torch.empty(capacity(field.shape), dtype=torch.uint8, device=field.device)
    used = torch.zeros(1, dtype=torch.int64, device=field.device)
    _check(_decl().ccb_sz_compress(field.data_ptr(), nx, ny, nz, eb, buf.data_ptr(), used.data_ptr(), _stream()))
    return buf, used


def decompress(buf: torch.Tensor, shape, eb: float) -> torch.Tensor:
    nz, ny, nx = shape
    out = torch.empty(shape, dtype=torch.float32, device=buf.device)
    _check(_decl().ccb_sz_decompress(buf.data_ptr(), nx, ny, nz, eb, out.data_ptr(), _stream()))
    return out


def all_gather(comm: Communicator, send, recv, eb: float, used: torch.Tensor | None = None):
    """Error-bounded AllGather of one [nz, ny, nx] field per rank; recv: [nranks, nz, ny, nx]."""
    return _collective(comm, send, recv, eb, -1, used)


def broadcast(comm: Communicator, send, recv, eb: float, root: int = 0, used: torch.Tensor | None = None):
    return _collective(comm, send, recv, eb, root, used)


def _collective(comm, send, recv, eb, root, used):
    sp, st = comm._ptrs(send, "send")
    rp, _ = comm._ptrs(recv, "recv")
    nz, ny, nx = st[0].shape[-3:]
    _check(_decl().ccb_sz_collective(comm._h, sp, rp, nx, ny, nz, eb, root, used.data_ptr() if used is not None else None,
                                     _stream()))
    return recv


# -------------------------------------------------------------- container --
# A compressed buffer in device memory is a row of fixed-capacity group slots
# ([8 x u32 tile sizes][tiles back to back], GROUP_STRIDE bytes each), mostly empty. For
# storage or for transports that want one contiguous message it is packed into a
# self-describing container:
#   [u32 magic 'CCSZ'][u32 version = 2][u32 nx][u32 ny][u32 nz][f32 eb][f32 step][u32 ngroups]
#   [u64 payload bytes][u32 used bytes of each group (header included)] [the used bytes of every group]
MAGIC, VERSION = 0x5A534343, 2
GROUP_STRIDE, GROUP_HEADER, HEADER_BYTES = 66112, 32, 40


def to_container(buf: torch.Tensor, shape, eb: float) -> torch.Tensor:
    """Packs the group slots of `buf` (as returned by compress) into one contiguous uint8
    tensor on the same device. Plain tensor operations, no extra kernel."""
    nz, ny, nx = shape
    ngroups = buf.numel() // GROUP_STRIDE
    slots = buf.view(ngroups, GROUP_STRIDE)
    sizes = slots[:, :GROUP_HEADER].contiguous().view(torch.int32).to(torch.int64).sum(dim=1) + GROUP_HEADER
    keep = torch.arange(GROUP_STRIDE, device=buf.device).unsqueeze(0) < sizes.unsqueeze(1)
    payload = slots[keep]
    step = torch.tensor(2.0 * eb, dtype=torch.float32) * (1 - 2.0 ** -10)
    head = torch.zeros(HEADER_BYTES, dtype=torch.uint8)
    head[0:20].view(torch.int32).copy_(torch.tensor([MAGIC, VERSION, nx, ny, nz], dtype=torch.int32))
    head[20:28].view(torch.float32).copy_(torch.tensor([eb, step.item()], dtype=torch.float32))
    head[28:32].view(torch.int32).copy_(torch.tensor([ngroups], dtype=torch.int32))
    head[32:40].view(torch.int64).copy_(torch.tensor([payload.numel()], dtype=torch.int64))
    return torch.cat([head.to(buf.device), sizes.to(torch.int32).view(torch.uint8), payload])


def from_container(blob: torch.Tensor):
    """Inverse of to_container: returns (buffer of group slots, shape, eb)."""
    head = blob[:HEADER_BYTES].cpu()
    magic, version, nx, ny, nz = head[0:20].view(torch.int32).tolist()
    if magic != MAGIC or version != VERSION:
        raise ValueError(f"not a ccb-sz v{VERSION} container (magic {magic:#x}, version {version})")
    eb = head[20:24].view(torch.float32).item()
    ngroups = head[28:32].view(torch.int32).item()
    nbytes = head[32:40].view(torch.int64).item()
    if ngroups * GROUP_STRIDE != capacity((nz, ny, nx)):
        raise ValueError("container header does not match its dimensions")
    sizes = blob[HEADER_BYTES:HEADER_BYTES + 4 * ngroups].contiguous().view(torch.int32).to(torch.int64)
    payload = blob[HEADER_BYTES + 4 * ngroups:]
    if payload.numel() != nbytes or int(sizes.sum().item()) != nbytes or int(sizes.max().item()) > GROUP_STRIDE:
        raise ValueError("container payload is damaged")
    buf = torch.zeros(ngroups, GROUP_STRIDE, dtype=torch.uint8, device=blob.device)
    keep = torch.arange(GROUP_STRIDE, device=blob.device).unsqueeze(0) < sizes.unsqueeze(1)
    buf[keep] = payload
    return buf.view(-1), (nz, ny, nx), eb


def save(path, field: torch.Tensor, eb: float) -> int:
    """Compresses `field` and writes the container to `path`; returns the file size."""
    buf, _ = compress(field, eb)
    blob = to_container(buf, field.shape, eb).cpu().numpy()
    blob.tofile(path)
    return int(blob.size)


def load(path, device="cuda") -> torch.Tensor:
    blob = torch.from_numpy(np.fromfile(path, dtype=np.uint8)).to(device)
    buf, shape, eb = from_container(blob)
    return decompress(buf, shape, eb)


# ------------------------------------------------------------------ oracle --
def restate(field: np.ndarray, eb: float):
    """NumPy restatement: returns (reconstruction fp32, packed bytes per the format)."""
    x = field.astype(np.float32)
    two_eb = np.float32(2.0) * np.float32(eb) * (np.float32(1.0) - np.float32(2.0 ** -10))
    inv = np.float32(1.0) / two_eb
    half = np.float32(0.5) * two_eb
    q = np.rint(x * inv).astype(np.int64)
    r = (q.astype(np.float32) * two_eb).astype(np.float32)
    q = q + ((x - r) > half) - ((r - x) > half)
    recon = (q.astype(np.float32) * two_eb).astype(np.float32)
    nz, ny, nx = x.shape
    pz, py, px = (-nz) % TZ, (-ny) % TY, (-nx) % TX
    qp = np.pad(q, ((0, pz), (0, py), (0, px)))
    Z, Y, X = qp.shape
    t = qp.reshape(Z // TZ, TZ, Y // TY, TY, X // TX, TX).transpose(0, 2, 4, 1, 3, 5)  # [tz,ty,tx, z,y,x]
    d = t.copy()
    d[..., 1:, :, :] -= t[..., :-1, :, :]
    d2 = d.copy()
    d2[..., :, 1:, :] -= d[..., :, :-1, :]
    d3 = d2.copy()
    d3[..., :, :, 1:] -= d2[..., :, :, :-1]
    u = ((d3 << 1) ^ (d3 >> 63)).astype(np.uint64) & np.uint64(0xFFFFFFFF)
    # a packing row is element e (of 8 consecutive x) over the 8 lines x 4 segments of a plane
    mx = u.reshape(u.shape[:-2] + (TY, TX // 8, 8)).max(axis=(-2, -3))  # [..., z, e]
    w = np.where(mx > 0, np.floor(np.log2(np.maximum(mx, 1).astype(np.float64))).astype(np.int64) + 1, 0)
    tile_bytes = 64 + 4 * w.sum(axis=(-1, -2))
    tile_bytes = (tile_bytes + 15) // 16 * 16
    return recon, int(tile_bytes.sum())
