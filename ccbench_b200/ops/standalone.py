"""Stand-alone codec kernels on local memory (no communicator): what the compression
hook ABIs are built from. Wire layout of `count` elements: pad = count rounded up to 512,
[payload: pad elements][scales: pad / group entries]."""
from __future__ import annotations

import ctypes

import torch

from .. import constants as K
from .._lib import lib
from ..comm import _check, _DTYPES, wire_bytes


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _p(t: torch.Tensor):
    return ctypes.c_void_p(t.data_ptr())


def encode(x: torch.Tensor, codec: str) -> torch.Tensor:
    """Returns the wire bytes (uint8 tensor) of a contiguous CUDA tensor."""
    wire = torch.empty(wire_bytes(codec, x.dtype, x.numel()), dtype=torch.uint8, device=x.device)
    _check(lib().ccb_encode(K.CODECS[codec], _DTYPES[x.dtype], _p(x), ctypes.c_uint64(x.numel()), _p(wire), _stream()))
    return wire


def decode(wire: torch.Tensor, codec: str, count: int, dtype: torch.dtype) -> torch.Tensor:
    out = torch.empty(count, dtype=dtype, device=wire.device)
    _check(lib().ccb_decode(K.CODECS[codec], _DTYPES[dtype], _p(wire), ctypes.c_uint64(count), _p(out), _stream()))
    return out


def decode_reduce(wire: torch.Tensor, codec: str, inout: torch.Tensor) -> torch.Tensor:
    """inout += decode(wire), one kernel."""
    _check(lib().ccb_decode_reduce(K.CODECS[codec], _DTYPES[inout.dtype], _p(wire), ctypes.c_uint64(inout.numel()), _p(inout),
                                   _stream()))
    return inout


def reduce_recode(wires, codec: str, count: int) -> torch.Tensor:
    """encode(sum_k decode(wires[k])) without leaving the compressed domain in memory."""
    arr = (ctypes.c_void_p * len(wires))(*[w.data_ptr() for w in wires])
    out = torch.empty_like(wires[0])
    _check(lib().ccb_reduce_recode(K.CODECS[codec], arr, len(wires), ctypes.c_uint64(count), _p(out), _stream()))
    return out


def refwire_bytes(count: int, group: int) -> int:
    return (count + group - 1) // group * 4 + count


def refwire_encode(x: torch.Tensor, group: int = 256) -> torch.Tensor:
    """The reference wrapper's int8 wire: [f32 127/absmax per group][int8 x count]."""
    wire = torch.empty(refwire_bytes(x.numel(), group), dtype=torch.uint8, device=x.device)
    _check(lib().ccb_refwire_encode(_DTYPES[x.dtype], _p(x), ctypes.c_uint64(x.numel()), group, _p(wire), _stream()))
    return wire


def refwire_decode(wire: torch.Tensor, count: int, dtype: torch.dtype, group: int = 256) -> torch.Tensor:
    out = torch.empty(count, dtype=dtype, device=wire.device)
    _check(lib().ccb_refwire_decode(_DTYPES[dtype], _p(wire), ctypes.c_uint64(count), group, _p(out), _stream()))
    return out
