"""Synthetic, seeded inputs of the five benchmark configurations (harness only).

The reference feeds its benchmarks from rank patterns or from captured training
tensors tiled into .f32 files (scripts/intermediate/generate_iter_datasets.py,
run_codes/benchmark-core/src/utils.c:162-223); with no datasets available the
shapes and distributions are generated here instead."""
from __future__ import annotations


import torch


def gradient_like(count: int, dtype=torch.bfloat16, seed: int = 0, device="cpu", scale: float = 1e-3,
                  outlier_frac: float = 1e-3, outlier_gain: float = 100.0) -> torch.Tensor:
    """Laplace(0, scale) values with `outlier_frac` of the entries multiplied by `outlier_gain`."""
    g = torch.Generator(device=device).manual_seed(1234 + seed)
    out = torch.empty(count, dtype=dtype, device=device)
    step = 1 << 24
    for lo in range(0, count, step):
        n = min(step, count - lo)
        u = torch.rand(n, generator=g, device=device) - 0.5
        v = -scale * torch.sign(u) * torch.log1p(-2 * u.abs().clamp_(max=0.4999999))
        mask = torch.rand(n, generator=g, device=device) < outlier_frac
        v = torch.where(mask, v * outlier_gain, v)
        out[lo:lo + n] = v.to(dtype)
    return out


def uniform_pm1(count: int, dtype=torch.float32, seed: int = 0, device="cpu") -> torch.Tensor:
    g = torch.Generator(device=device).manual_seed(99 + seed)
    return (torch.rand(count, generator=g, device=device) * 2 - 1).to(dtype)


def normal(count: int, dtype=torch.float32, seed: int = 0, device="cpu") -> torch.Tensor:
    g = torch.Generator(device=device).manual_seed(seed)
    return torch.randn(count, generator=g, device=device).to(dtype)


def smooth_field(n: int = 512, seed: int = 0, device="cpu", bumps: int = 64, noise: float = 1e-3) -> torch.Tensor:
    """n^3 fp32 field: `bumps` Gaussian bumps (sigma 8-64 voxels at n=512, amplitude
    N(0,1)) plus seeded white noise. Separable evaluation keeps it O(bumps * n^3)."""
    g = torch.Generator(device="cpu").manual_seed(777 + seed)
    centers = torch.rand(bumps, 3, generator=g) * n
    sig = (8 + 56 * torch.rand(bumps, generator=g)) * (n / 512)
    amp = torch.randn(bumps, generator=g)
    ax = torch.arange(n, dtype=torch.float32, device=device)
    field = torch.zeros(n, n, n, device=device)
    for b in range(bumps):
        gx = torch.exp(-0.5 * ((ax - centers[b, 0].item()) / sig[b].item()) ** 2)
        gy = torch.exp(-0.5 * ((ax - centers[b, 1].item()) / sig[b].item()) ** 2)
        gz = torch.exp(-0.5 * ((ax - centers[b, 2].item()) / sig[b].item()) ** 2)
        field += amp[b].item() * gz[:, None, None] * gy[None, :, None] * gx[None, None, :]
    gd = torch.Generator(device=device).manual_seed(4242 + seed)
    field += noise * torch.randn(n, n, n, generator=gd, device=device)
    return field


def moe_routing(tokens: int, experts: int, topk: int = 2, seed: int = 0, device="cpu"):
    """Top-k routing from seeded uniform logits: (expert ids [tokens, topk], gates [tokens, topk])."""
    g = torch.Generator(device=device).manual_seed(31337 + seed)
    logits = torch.rand(tokens, experts, generator=g, device=device)
    w, idx = torch.topk(torch.softmax(logits, dim=-1), topk, dim=-1)
    return idx.to(torch.int32), (w / w.sum(-1, keepdim=True)).float()
