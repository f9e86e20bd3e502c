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
