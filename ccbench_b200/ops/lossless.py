"""Lossless float codec: the GPU entry points of libccb.so and a NumPy restatement of the
same container, used as the oracle of the GPU tests and on hosts without a GPU.

Container (see include/ccb/ccb_lossless.h): a 32-byte header, then one fixed-stride slot
per 4096 values; in a slot the sign and mantissa bits are raw planes and the exponent of
every value is stored relative to the minimum of its 512-value block in as many bit planes
as the block needs. Role in the reference: DietGPU's float codec
(userconfig/wrapper_code_examples/compression/dietgpu/dietgpu.cu:32-103) and the ratio
measurement of scripts/intermediate/test_dietgpu_compress.py."""
from __future__ import annotations

import ctypes

import numpy as np

MAGIC = 0x4C424343
TILE, BLOCK, HEADER = 4096, 512, 32
# dtype code -> (bytes per element, exponent shift, exponent bits, mantissa bits)
_FMT = {0: (4, 23, 8, 23), 1: (2, 7, 8, 7), 2: (2, 10, 5, 10)}


def slot_bytes(dtype_code: int) -> int:
    return 32 + TILE * _FMT[dtype_code][0]


def max_bytes(dtype_code: int, count: int) -> int:
    return HEADER + (count + TILE - 1) // TILE * slot_bytes(dtype_code)


def _split(bits: np.ndarray, code: int):
    esz, sh, eb, mb = _FMT[code]
    b = bits.astype(np.uint32)
    key = (b >> sh) & ((1 << eb) - 1)
    sign = b >> (8 * esz - 1)
    rest = (b & ((1 << mb) - 1)) | (sign << mb)
    return key, rest


def _join(key: np.ndarray, rest: np.ndarray, code: int) -> np.ndarray:
    esz, sh, eb, mb = _FMT[code]
    return ((rest >> mb) << (8 * esz - 1)) | (key << sh) | (rest & ((1 << mb) - 1))


def _ballots(v: np.ndarray, bit: int) -> np.ndarray:
    """v: [32 lanes, 16 values] -> 16 words, word j bit l = bit `bit` of v[l, j]."""
    b = ((v >> bit) & 1).astype(np.uint64)
    return (b << np.arange(32, dtype=np.uint64)[:, None]).sum(0).astype(np.uint32)


def np_encode(bits: np.ndarray, code: int) -> np.ndarray:
    """bits: the values' bit patterns (uint32 for f32, uint16 otherwise). Returns the
    container as uint8 of max_bytes() length; bytes past a slot's used prefix are zero."""
    esz = _FMT[code][0]
    count = bits.size
    ntiles = (count + TILE - 1) // TILE
    out = np.zeros(max_bytes(code, count), dtype=np.uint8)
    padded = np.zeros(ntiles * TILE, dtype=np.uint32)
    padded[:count] = bits
    total = HEADER
    rest_bytes = {0: 3 * TILE, 1: TILE, 2: TILE + 3 * TILE // 8}[code]
    for t in range(ntiles):
        slot = out[HEADER + t * slot_bytes(code):HEADER + (t + 1) * slot_bytes(code)]
        key, rest = _split(padded[t * TILE:(t + 1) * TILE], code)
        widths, kmins, planes = [], [], []
        for blk in range(TILE // BLOCK):
            k = key[blk * BLOCK:(blk + 1) * BLOCK]
            kmin, kmax = int(k.min()), int(k.max())
            w = 0 if kmax == kmin else int(kmax - kmin).bit_length()
            widths.append(w)
            kmins.append(kmin)
            d = (k - kmin).reshape(32, 16)
            planes.append(np.concatenate([_ballots(d, p) for p in range(w)]) if w else np.zeros(0, np.uint32))
        r = rest
        if code == 0:
            for p in range(3):
                slot[32 + p * TILE:32 + (p + 1) * TILE] = ((r >> (8 * p)) & 0xff).astype(np.uint8)
        else:
            slot[32:32 + TILE] = (r & 0xff).astype(np.uint8)
            if code == 2:
                words = np.concatenate([np.concatenate([_ballots(r[b * BLOCK:(b + 1) * BLOCK].reshape(32, 16), 8 + p) for p in range(3)])
                                        for b in range(TILE // BLOCK)])
                slot[32 + TILE:32 + rest_bytes] = words.view(np.uint8)
        exp = np.concatenate(planes).astype(np.uint32)
        used = 32 + rest_bytes + exp.size * 4
        slot[32 + rest_bytes:used] = exp.view(np.uint8)
        slot[0:4] = np.array([used], np.uint32).view(np.uint8)
        slot[4:12] = np.array(widths, np.uint8)
        slot[12:20] = np.array(kmins, np.uint8)
        total += used
    out[0:8] = np.array([MAGIC, code], np.uint32).view(np.uint8)
    out[8:24] = np.array([count, total], np.uint64).view(np.uint8)
    return out


def np_decode(buf: np.ndarray, code: int | None = None) -> np.ndarray:
    """Container -> bit patterns (uint32 for f32, uint16 otherwise)."""
    magic, dcode = buf[0:8].view(np.uint32)
    assert magic == MAGIC, "not a lossless float container"
    code = int(dcode) if code is None else code
    count = int(buf[8:16].view(np.uint64)[0])
    esz = _FMT[code][0]
    rest_bytes = {0: 3 * TILE, 1: TILE, 2: TILE + 3 * TILE // 8}[code]
    ntiles = (count + TILE - 1) // TILE
    bits = np.zeros(ntiles * TILE, dtype=np.uint32)
    lanes = np.arange(32, dtype=np.uint32)[:, None]
    for t in range(ntiles):
        slot = buf[HEADER + t * slot_bytes(code):HEADER + (t + 1) * slot_bytes(code)]
        widths, kmins = slot[4:12].astype(int), slot[12:20].astype(np.uint32)
        if code == 0:
            rest = sum(slot[32 + p * TILE:32 + (p + 1) * TILE].astype(np.uint32) << (8 * p) for p in range(3))
        else:
            rest = slot[32:32 + TILE].astype(np.uint32)
            if code == 2:
                words = slot[32 + TILE:32 + rest_bytes].view(np.uint32).reshape(TILE // BLOCK, 3, 16)
                for b in range(TILE // BLOCK):
                    for p in range(3):
                        rest[b * BLOCK:(b + 1) * BLOCK] |= (((words[b, p][None, :] >> lanes) & 1) << (8 + p)).reshape(-1)
        exp = slot[32 + rest_bytes:32 + rest_bytes + 64 * int(widths.sum())].view(np.uint32)
        key = np.zeros(TILE, dtype=np.uint32)
        off = 0
        for b in range(TILE // BLOCK):
            w = int(widths[b])
            pl = exp[off * 16:(off + w) * 16].reshape(w, 16)
            d = np.zeros((32, 16), dtype=np.uint32)
            for p in range(w):
                d |= ((pl[p][None, :] >> lanes) & 1) << p
            key[b * BLOCK:(b + 1) * BLOCK] = d.reshape(-1) + kmins[b]
            off += w
        bits[t * TILE:(t + 1) * TILE] = _join(key, rest, code)
    return bits[:count].astype(np.uint32 if esz == 4 else np.uint16)


def used_bytes_np(buf: np.ndarray) -> int:
    return int(buf[16:24].view(np.uint64)[0])


# ------------------------------------------------------------------ GPU entry points --
def _gpu():
    import torch

    from .. import constants as K
    from .._lib import lib
    from ..comm import _DTYPES, _check

    L = lib()
    L.ccb_lossless_max_bytes.restype = ctypes.c_uint64
    L.ccb_lossless_max_bytes.argtypes = [ctypes.c_int, ctypes.c_uint64]
    L.ccb_lossless_encode.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_uint64, ctypes.c_void_p, ctypes.c_void_p]
    L.ccb_lossless_decode.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_uint64, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p]
    L.ccb_lossless_used_bytes.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_uint64), ctypes.c_void_p]
    return torch, L, _DTYPES, _check


def encode(x):
    """x: contiguous CUDA tensor (float32, bfloat16 or float16) -> container (uint8 CUDA tensor)."""
    torch, L, DT, check = _gpu()
    out = torch.empty(int(L.ccb_lossless_max_bytes(DT[x.dtype], x.numel())), dtype=torch.uint8, device=x.device)
    check(L.ccb_lossless_encode(DT[x.dtype], x.data_ptr(), x.numel(), out.data_ptr(), torch.cuda.current_stream().cuda_stream))
    return out


def decode(comp, count: int, dtype, out=None, accumulate: bool = False):
    torch, L, DT, check = _gpu()
    out = torch.empty(count, dtype=dtype, device=comp.device) if out is None else out
    check(L.ccb_lossless_decode(DT[dtype], comp.data_ptr(), count, out.data_ptr(), 1 if accumulate else 0,
                                torch.cuda.current_stream().cuda_stream))
    return out


def used_bytes(comp) -> int:
    torch, L, DT, check = _gpu()
    v = ctypes.c_uint64(0)
    check(L.ccb_lossless_used_bytes(comp.data_ptr(), ctypes.byref(v), torch.cuda.current_stream().cuda_stream))
    return int(v.value)


def ratio(x) -> float:
    """Raw bytes / bytes that carry information, for a CUDA tensor."""
    return x.numel() * x.element_size() / used_bytes(encode(x))
