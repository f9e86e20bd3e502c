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


def launch_path() -> int:
    """How the last collective launch went: 1 = cluster + cooperative attributes accepted
    together, 2 = the driver refused the pair and the cluster attribute was used alone, 0 =
    no collective launched yet."""
    return int(_decl().ccb_sz_launch_path())


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


# ------------------------------------------------------------ CPU codec --
# The same format in NumPy, for hosts without a GPU (reading a stored field, checking a
# transfer) and as a second statement of the layout. Slow (seconds for 128^3): not a
# benchmark path.
_QMAX = float(1 << 22)


def _step(eb: float):
    two_eb = np.float32(2.0) * np.float32(eb) * (np.float32(1.0) - np.float32(2.0 ** -10))
    return two_eb, np.float32(1.0) / two_eb


def _tiles_of(a: np.ndarray):
    """[nz, ny, nx] -> [tiles, 8, 8, 32], zero-padded, tiles ordered x fastest."""
    nz, ny, nx = a.shape
    a = np.pad(a, ((0, (-nz) % TZ), (0, (-ny) % TY), (0, (-nx) % TX)))
    Z, Y, X = a.shape
    return a.reshape(Z // TZ, TZ, Y // TY, TY, X // TX, TX).transpose(0, 2, 4, 1, 3, 5).reshape(-1, TZ, TY, TX)


def _pack_tile_cpu(vals: np.ndarray, two_eb, inv, eb32) -> bytes:
    s = vals * inv
    bad = ~np.isfinite(vals).all() or not (np.abs(s) < _QMAX).all()
    if not bad:
        q = np.rint(s).astype(np.int64)
        r = q.astype(np.float32) * two_eb
        half = np.float32(0.5) * two_eb
        q = q + ((vals - r) > half) - ((r - vals) > half)
        bad = bool((np.abs(vals - q.astype(np.float32) * two_eb) > eb32).any())
    if bad:
        return bytes([255] + [0] * 63) + vals.astype("<f4").tobytes()
    d = q.copy()
    d[1:] -= q[:-1]
    d2 = d.copy()
    d2[:, 1:] -= d[:, :-1]
    d3 = d2.copy()
    d3[:, :, 1:] -= d2[:, :, :-1]
    u = ((d3 << 1) ^ (d3 >> 63)) & 0xFFFFFFFF
    rows = u.reshape(TZ, TY, TX // 8, 8).transpose(0, 3, 1, 2).reshape(TZ * 8, 32)   # row 8z+e, thread 4y+xq
    mx = rows.max(axis=1)
    widths = np.array([int(m).bit_length() for m in mx], dtype=np.uint8)
    out = bytearray(widths.tobytes())
    weights = (np.uint64(1) << np.arange(32, dtype=np.uint64))
    for row, w in zip(rows.astype(np.uint64), widths):
        for j in range(int(w)):
            out += int((((row >> np.uint64(j)) & np.uint64(1)) * weights).sum()).to_bytes(4, "little")
    out += bytes((-len(out)) % 16)
    return bytes(out)


def encode_cpu(field: np.ndarray, eb: float) -> np.ndarray:
    """Compresses a [nz, ny, nx] fp32 array into the container format (uint8 array)."""
    x = np.ascontiguousarray(field, dtype=np.float32)
    nz, ny, nx = x.shape
    two_eb, inv = _step(eb)
    eb32 = np.float32(eb)
    tiles = _tiles_of(x)
    packed = [_pack_tile_cpu(t, two_eb, inv, eb32) for t in tiles]
    ngroups = (len(packed) + 7) // 8
    groups, used = [], []
    for g in range(ngroups):
        mine = packed[8 * g:8 * g + 8]
        sizes = np.zeros(8, dtype="<u4")
        sizes[:len(mine)] = [len(p) for p in mine]
        groups.append(sizes.tobytes() + b"".join(mine))
        used.append(len(groups[-1]))
    payload = b"".join(groups)
    head = np.zeros(HEADER_BYTES, dtype=np.uint8)
    head[0:20].view("<i4")[:] = [MAGIC, VERSION, nx, ny, nz]
    head[20:28].view("<f4")[:] = [eb32, two_eb]
    head[28:32].view("<i4")[:] = [ngroups]
    head[32:40].view("<i8")[:] = [len(payload)]
    return np.concatenate([head, np.array(used, dtype="<u4").view(np.uint8), np.frombuffer(payload, dtype=np.uint8)])


def decode_cpu(blob: np.ndarray) -> np.ndarray:
    """Inverse of encode_cpu (and of to_container on a GPU-compressed buffer)."""
    blob = np.asarray(blob, dtype=np.uint8)
    magic, version, nx, ny, nz = blob[0:20].view("<i4").tolist()
    if magic != MAGIC or version != VERSION:
        raise ValueError("not a ccb-sz v2 container")
    two_eb = blob[24:28].view("<f4")[0]
    ngroups = int(blob[28:32].view("<i4")[0])
    used = blob[HEADER_BYTES:HEADER_BYTES + 4 * ngroups].view("<u4").astype(np.int64)
    body = blob[HEADER_BYTES + 4 * ngroups:]
    if int(used.sum()) != body.size:
        raise ValueError("container payload is damaged")
    tx, ty, tz = -(-nx // TX), -(-ny // TY), -(-nz // TZ)
    ntiles = tx * ty * tz
    out = np.zeros((tz * TZ, ty * TY, tx * TX), dtype=np.float32)
    shifts = np.arange(32, dtype=np.uint64)
    pos = 0
    for g in range(ngroups):
        grp = body[pos:pos + int(used[g])]
        pos += int(used[g])
        sizes = grp[:GROUP_HEADER].view("<u4")
        off = GROUP_HEADER
        for k in range(8):
            tile = 8 * g + k
            if tile >= ntiles or sizes[k] == 0:
                continue
            t = grp[off:off + int(sizes[k])]
            off += int(sizes[k])
            if t[0] == 255:
                vals = t[64:64 + 4 * TZ * TY * TX].view("<f4").reshape(TZ, TY, TX)
            else:
                widths = t[:64]
                words = t[64:].view("<u4").astype(np.uint64)
                rows = np.zeros((TZ * 8, 32), dtype=np.uint64)
                w0 = 0
                for r, w in enumerate(widths):
                    for j in range(int(w)):
                        rows[r] |= ((words[w0 + j] >> shifts) & np.uint64(1)) << np.uint64(j)
                    w0 += int(w)
                u = rows.reshape(TZ, 8, TY, TX // 8).transpose(0, 2, 3, 1).reshape(TZ, TY, TX).astype(np.int64)
                d = (u >> 1) ^ -(u & 1)
                q = d.cumsum(axis=2).cumsum(axis=1).cumsum(axis=0)
                vals = q.astype(np.float32) * two_eb
            z0, y0, x0 = tile // (tx * ty) * TZ, tile // tx % ty * TY, tile % tx * TX
            out[z0:z0 + TZ, y0:y0 + TY, x0:x0 + TX] = vals
    return out[:nz, :ny, :nx].copy()


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


def selfcheck(n: int = 48, eb_rel: float = 1e-3, device: str = "cuda") -> dict:
    """Cross-check of the two implementations of the format on a small field: what the GPU
    packs, the NumPy decoder must read back to the GPU decoder's values, and what the NumPy
    encoder packs, the GPU must decode to the NumPy decoder's values.
    `python -m ccbench_b200.ops.sz` prints the outcome."""
    from ..models.workloads import smooth_field

    f = smooth_field(n, seed=3, device=device)[:, : n - 5, : n - 3].contiguous()
    eb = eb_rel * (f.max() - f.min()).item()
    buf, _ = compress(f, eb)
    gpu = decompress(buf, f.shape, eb).cpu().numpy()
    blob = to_container(buf, f.shape, eb).cpu().numpy()
    cpu_from_gpu = decode_cpu(blob)
    blob_cpu = encode_cpu(f.cpu().numpy(), eb)
    buf2, shape2, eb2 = from_container(torch.from_numpy(blob_cpu).to(device))
    gpu_from_cpu = decompress(buf2, shape2, eb2).cpu().numpy()
    return {"gpu_pack_cpu_unpack": bool(np.array_equal(cpu_from_gpu, gpu)),
            "cpu_pack_gpu_unpack": bool(np.array_equal(gpu_from_cpu, decode_cpu(blob_cpu))),
            "same_bytes": bool(blob.size == blob_cpu.size and np.array_equal(blob, blob_cpu)),
            "bytes": int(blob.size)}


if __name__ == "__main__":
    import json

    print(json.dumps(selfcheck()))
