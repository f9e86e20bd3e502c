"""Plain PyTorch fp32 restatements of the wire codecs and of each algorithm's
quantisation points. They are the oracles the CUDA kernels are tested against and
the CPU path of the 2-rank gloo benchmark; nothing here is on a GPU hot path.

Codec definitions (identical to csrc/kernels/ccb_codec.cuh):
  int8  : per group of G values, scale = absmax/127, q = rint(x * (127/absmax))
  int4  : per group of 128 values, scale = absmax/7, q = rint(x * (7/absmax)), two per byte
  fp8   : per 32 values, scale 2^e with e the smallest integer such that
          absmax * 2^-e <= 448; q = e4m3(x * 2^-e) (round to nearest even)
The reference's int8 codec stores the reciprocal 127/absmax instead
(plain_nccl_compress.cu:141-177); `int8_encode_reference_wire` produces that layout.
"""
from __future__ import annotations

import torch

PAD = 512


def _pad_to(x: torch.Tensor, m: int) -> torch.Tensor:
    n = x.numel()
    r = (-n) % m
    if r:
        x = torch.cat([x.reshape(-1), x.new_zeros(r)])
    return x.reshape(-1)


def int8_encode(x: torch.Tensor, group: int = 128):
    """Returns (q int8 [n_pad], scale fp32 [n_pad/group]) for fp32 x (padded with zeros)."""
    xf = _pad_to(x.float(), group).reshape(-1, group)
    m = xf.abs().amax(dim=1, keepdim=True)
    # tensor / tensor so that both quotients are single IEEE divisions like the kernel's
    # (`127.0 / m` and `m / 127.0` with a Python scalar go through a reciprocal)
    c127 = torch.full_like(m, 127.0)
    inv = torch.where(m > 0, c127 / m.clamp_min(torch.finfo(torch.float32).tiny), torch.zeros_like(m))
    q = torch.round(xf * inv).clamp_(-127, 127).to(torch.int8)
    return q.reshape(-1), (m / c127).reshape(-1)


def int8_decode(q: torch.Tensor, scale: torch.Tensor, group: int = 128) -> torch.Tensor:
    return (q.reshape(-1, group).float() * scale.reshape(-1, 1)).reshape(-1)


def int4_roundtrip(x: torch.Tensor, group: int = 128) -> torch.Tensor:
    """Symmetric 4-bit integers (-7..7), fp32 scale = absmax / 7 per group."""
    xf = _pad_to(x.float(), group).reshape(-1, group)
    m = xf.abs().amax(dim=1, keepdim=True)
    c7 = torch.full_like(m, 7.0)
    inv = torch.where(m > 0, c7 / m.clamp_min(torch.finfo(torch.float32).tiny), torch.zeros_like(m))
    q = torch.round(xf * inv).clamp_(-7, 7)
    return (q * (m / c7)).reshape(-1)[: x.numel()].reshape(x.shape)


def int8_roundtrip(x: torch.Tensor, group: int = 128) -> torch.Tensor:
    q, s = int8_encode(x, group)
    return int8_decode(q, s, group)[: x.numel()].reshape(x.shape)


def int8_encode_reference_wire(x: torch.Tensor, group: int = 256):
    """The reference wrapper's wire: reciprocal scales (127/absmax, 1.0 when the group
    is all ~0) followed by the int8 payload."""
    xf = _pad_to(x.float(), group).reshape(-1, group)
    m = xf.abs().amax(dim=1, keepdim=True)
    inv = torch.where(m < 1e-10, torch.ones_like(m), torch.full_like(m, 127.0) / m.clamp_min(1e-30))
    q = torch.round(xf * inv).clamp_(-128, 127).to(torch.int8)
    return inv.reshape(-1), q.reshape(-1)[: x.numel()]


def ue8m0_exponent(absmax: torch.Tensor) -> torch.Tensor:
    """Smallest e (int32) with absmax * 2^-e <= 448, clamped to [-126, 126]."""
    bits = absmax.float().contiguous().view(torch.int32)
    e = (bits >> 23) - 127 - 8 + ((bits & 0x7FFFFF) > 0x600000).to(torch.int32)
    return e.clamp_(-126, 126)


def fp8_encode(x: torch.Tensor):
    xf = _pad_to(x.float(), 32).reshape(-1, 32)
    e = ue8m0_exponent(xf.abs().amax(dim=1, keepdim=True))
    inv = torch.ldexp(torch.ones_like(xf[:, :1]), -e)
    q = (xf * inv).to(torch.float8_e4m3fn)
    return q.reshape(-1), (e + 127).to(torch.uint8).reshape(-1)


def fp8_decode(q: torch.Tensor, ebyte: torch.Tensor) -> torch.Tensor:
    e = ebyte.to(torch.int32).reshape(-1, 1) - 127
    v = q.reshape(-1, 32).float()
    return torch.ldexp(v, e.expand_as(v)).reshape(-1)


def fp8_roundtrip(x: torch.Tensor) -> torch.Tensor:
    q, e = fp8_encode(x)
    return fp8_decode(q, e)[: x.numel()].reshape(x.shape)


def roundtrip(x: torch.Tensor, codec: str, dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """decode(encode(x)) in fp32 for the named codec; 'none' rounds to the wire dtype."""
    if codec == "int8":
        return int8_roundtrip(x, 128)
    if codec == "int8_g256":
        return int8_roundtrip(x, 256)
    if codec == "fp8":
        return fp8_roundtrip(x)
    if codec == "int4":
        return int4_roundtrip(x)
    if codec == "none":
        return x.float().to(dtype).float()
    raise ValueError(codec)


def wire_ratio(codec: str, dtype: torch.dtype) -> float:
    """Raw bytes / wire bytes of one message."""
    es = torch.empty((), dtype=dtype).element_size()
    per = {"none": es, "int8": 1 + 4 / 128, "int8_g256": 1 + 4 / 256, "fp8": 1 + 1 / 32, "int4": 0.5 + 4 / 128}[codec]
    return es / per


# ------------------------------------------------------------------ algorithms --
def _shards(count: int, n: int, m: int = PAD):
    se = -(-(-(-count // n)) // m) * m
    return se, [(min(s * se, count), min((s + 1) * se, count)) for s in range(n)]


def simulate_all_reduce(xs, codec: str, algo: str = "twoshot", dtype=None, ef=None):
    """What the fused kernels compute, restated with torch ops: returns one fp32 result
    per rank (all equal). xs: list of per-rank tensors. ef: optional list of fp32
    residual tensors, updated in place."""
    n = len(xs)
    dtype = dtype or xs[0].dtype
    X = [x.float().reshape(-1) for x in xs]
    count = X[0].numel()
    rt = lambda v: roundtrip(v, codec, dtype)
    out = torch.empty(count)

    def quant(rank, lo, hi, v):
        if ef is not None:
            v = v + ef[rank][lo:hi]
        d = rt(v)
        if ef is not None:
            ef[rank][lo:hi] = v - d
        return d

    if algo == "oneshot":
        acc = None
        for q in range(n):
            d = quant(q, 0, count, X[q])
            acc = d if acc is None else acc + d
        out = acc
    elif algo == "twoshot":
        se, sh = _shards(count, n)
        for r, (lo, hi) in enumerate(sh):
            if hi <= lo:
                continue
            acc = X[r][lo:hi].clone()
            for q in range(n):
                if q != r:
                    acc = acc + quant(q, lo, hi, X[q][lo:hi])
            out[lo:hi] = quant(r, lo, hi, acc)
    elif algo == "ring":
        se, sh = _shards(count, n)
        for c, (lo, hi) in enumerate(sh):
            if hi <= lo:
                continue
            # chunk c starts at rank c (step 0) and ends at rank c-1 after n-1 hops
            v = None
            for s in range(n):
                r = (c + s) % n
                t = X[r][lo:hi] if v is None else X[r][lo:hi] + v
                v = quant(r, lo, hi, t)
            out[lo:hi] = v
    elif algo == "tree":
        L = 0
        while (1 << L) < n:
            L += 1
        part = {}

        def up(r):
            tz = L if r == 0 else ((r & -r).bit_length() - 1)
            v = X[r].clone()
            for k in range(tz):
                if r + (1 << k) < n:
                    v = v + up(r + (1 << k))
            return quant(r, 0, count, v)

        out = up(0)
    else:
        raise ValueError(algo)
    return out.to(dtype).float()  # the kernels round the decoded fp32 to the user dtype on store
