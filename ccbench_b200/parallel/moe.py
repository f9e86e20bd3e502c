"""Expert-parallel token exchange (MoE): routing metadata in torch, data movement by
the fused dispatch / combine kernels (csrc/kernels/ccb_moe.cu). One expert per rank
group: expert e lives on rank e % nranks.

The reference only times a flat, equal-block AllToAll
(run_codes/benchmarks/nccl/alltoall/alltoall.c); this is the routed workload that
AlltoAll serves in MoE training, with per-destination fp8 compression."""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch

from .. import constants as K
from .._lib import lib
from ..comm import Communicator, _check, _code, _DTYPES


@dataclass
class Route:
    """Everything one rank needs for dispatch and combine."""
    perm: torch.Tensor        # int32 [T*k]: send order -> token row, grouped by destination rank
    dest_rank: torch.Tensor   # int32 [T*k]: destination rank of pair (t, k)
    pos: torch.Tensor         # int32 [T*k]: index of pair (t, k) inside the block sent to its destination
    gate: torch.Tensor        # fp32  [T*k]
    send_counts: torch.Tensor  # int64 [nranks]: rows this rank sends to each rank
    topk: int


def plan_route(expert_ids: torch.Tensor, gates: torch.Tensor, nranks: int) -> Route:
    """expert_ids, gates: [T, k]. Stable sort of the (t, k) pairs by destination rank."""
    T, k = expert_ids.shape
    dest = (expert_ids.reshape(-1).to(torch.int64) % nranks)
    order = torch.argsort(dest, stable=True)
    perm = (order // k).to(torch.int32)
    counts = torch.bincount(dest, minlength=nranks)
    starts = torch.cumsum(counts, 0) - counts
    pos = torch.empty(T * k, dtype=torch.int64, device=dest.device)
    pos[order] = torch.arange(T * k, device=dest.device) - starts[dest[order]]
    return Route(perm.contiguous(), dest.to(torch.int32).contiguous(), pos.to(torch.int32).contiguous(),
                 gates.reshape(-1).float().contiguous(), counts, k)


def _decl():
    L = lib()
    vp, pp, up = ctypes.c_void_p, ctypes.POINTER(ctypes.c_void_p), ctypes.POINTER(ctypes.c_uint64)
    L.ccb_moe_dispatch.argtypes = [vp, pp, pp, pp, up, ctypes.c_uint64, ctypes.c_int, ctypes.c_int, vp]
    L.ccb_moe_combine.argtypes = [vp, pp, pp, pp, pp, pp, up, ctypes.c_uint64, ctypes.c_int, ctypes.c_uint64, ctypes.c_int,
                                  ctypes.c_int, vp]
    return L


def _arr(ts):
    return (ctypes.c_void_p * len(ts))(*[t.data_ptr() for t in ts])


def _counts(count_matrix):
    flat = [int(v) for row in count_matrix for v in row]
    return (ctypes.c_uint64 * len(flat))(*flat)


def dispatch(comm: Communicator, x, recv, routes, count_matrix, *, codec="fp8"):
    """x, recv, routes: one per local rank. count_matrix[src][dst] rows (the same on every
    rank: all-gather the per-rank send_counts first). recv needs sum_s count[s][me] rows."""
    xs = [x] if isinstance(x, torch.Tensor) else list(x)
    rs = [recv] if isinstance(recv, torch.Tensor) else list(recv)
    rt = [routes] if isinstance(routes, Route) else list(routes)
    _check(_decl().ccb_moe_dispatch(comm._h, _arr(xs), _arr(rs), _arr([r.perm for r in rt]), _counts(count_matrix),
                                    xs[0].shape[-1], _DTYPES[xs[0].dtype], _code(codec, K.CODECS), comm._stream()))
    return recv


def combine(comm: Communicator, y, out, routes, count_matrix, *, codec="fp8"):
    ys = [y] if isinstance(y, torch.Tensor) else list(y)
    os_ = [out] if isinstance(out, torch.Tensor) else list(out)
    rt = [routes] if isinstance(routes, Route) else list(routes)
    _check(_decl().ccb_moe_combine(comm._h, _arr(ys), _arr(os_), _arr([r.dest_rank for r in rt]), _arr([r.pos for r in rt]),
                                   _arr([r.gate for r in rt]), _counts(count_matrix), os_[0].shape[0], rt[0].topk,
                                   os_[0].shape[-1], _DTYPES[os_[0].dtype], _code(codec, K.CODECS), comm._stream()))
    return out
