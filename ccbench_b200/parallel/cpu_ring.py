"""Ring AllReduce with a codec round trip at every hop, on CPU ranks over
torch.distributed (gloo): the algorithm of the reference's MPI wrapper
(userconfig/wrapper_code_examples/communication/plain_mpi_compress/plain_mpi_compress.c:
163-273) and of the fused ring kernel (csrc/kernels/ccb_ring.cuh), restated with torch ops.
It is the GPU-free member of the family: same chunking, same quantisation points, so its
result equals `ops.codecs.simulate_all_reduce(..., algo="ring")` bit for bit, and the
all-gather half forwards the final codes verbatim, so every rank ends with identical values.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..ops import codecs as C


def _encode(v: torch.Tensor, codec: str):
    if codec == "int8":
        q, s = C.int8_encode(v, 128)
        return [q, s]
    if codec == "fp8":
        q, e = C.fp8_encode(v)
        return [q.view(torch.uint8), e]
    if codec == "none":
        return [v.clone()]
    raise ValueError(f"codec {codec!r} has no CPU ring")


def _decode(parts, codec: str, n: int) -> torch.Tensor:
    if codec == "int8":
        return C.int8_decode(parts[0], parts[1], 128)[:n]
    if codec == "fp8":
        return C.fp8_decode(parts[0].view(torch.float8_e4m3fn), parts[1])[:n]
    return parts[0][:n]


def _like(parts):
    return [torch.empty_like(p) for p in parts]


def _exchange(send_parts, recv_parts, nxt: int, prv: int, group) -> None:
    reqs = [dist.isend(p, nxt, group=group) for p in send_parts]
    for p in recv_parts:
        dist.recv(p, prv, group=group)
    for q in reqs:
        q.wait()


def wire_bytes(parts) -> int:
    return sum(p.numel() * p.element_size() for p in parts)


def ring_all_reduce(x: torch.Tensor, codec: str = "int8", group=None, stats: dict | None = None) -> torch.Tensor:
    """Sum of `x` over the ranks of `group`; fp32 result of x's shape. `stats`, when given,
    receives the bytes this rank put on the wire and the raw bytes they stand for."""
    n, r = dist.get_world_size(group), dist.get_rank(group)
    flat = x.detach().float().reshape(-1)
    count = flat.numel()
    if n == 1:
        return C.roundtrip(flat, codec).reshape(x.shape)
    se, shards = C._shards(count, n)
    nxt, prv = (r + 1) % n, (r - 1) % n
    sent = raw = 0
    carried = None          # decoded running sum received at the previous hop
    codes = {}              # chunk -> final encoded parts (for the all-gather half)
    out = torch.empty(count)
    # reduce-scatter: n hops; at hop s this rank adds its own piece of chunk (r - s) to what
    # came in and re-encodes it. The hop s = n - 1 produces the final codes of chunk r + 1.
    for s in range(n):
        c = (r - s) % n
        lo, hi = shards[c]
        t = flat[lo:hi] if carried is None else flat[lo:hi] + carried
        parts = _encode(t, codec)
        if s == n - 1:
            codes[c] = parts
            break
        c_in = (r - s - 1) % n
        lo_in, hi_in = shards[c_in]
        recv = _like(_encode(torch.zeros(hi_in - lo_in), codec))
        _exchange(parts, recv, nxt, prv, group)
        sent += wire_bytes(parts)
        raw += (hi - lo) * 4
        carried = _decode(recv, codec, hi_in - lo_in)
    # all-gather: the final codes travel n - 1 hops unchanged; every rank decodes the same bytes
    have = (r + 1) % n
    for k in range(n - 1):
        lo, hi = shards[have]
        c_in = (have - 1) % n
        lo_in, hi_in = shards[c_in]
        recv = _like(_encode(torch.zeros(hi_in - lo_in), codec))
        _exchange(codes[have], recv, nxt, prv, group)
        sent += wire_bytes(codes[have])
        raw += (hi - lo) * 4
        codes[c_in] = recv
        have = c_in
    for c, parts in codes.items():
        lo, hi = shards[c]
        out[lo:hi] = _decode(parts, codec, hi - lo)
    if stats is not None:
        stats.update(wire_bytes=sent, raw_bytes=raw)
    return out.reshape(x.shape)
