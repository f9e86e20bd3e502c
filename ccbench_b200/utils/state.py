"""Training state of the compressed collectives that outlives a process: the error-feedback
residual. It is what the codec dropped in earlier calls and still owes the sum, so a job
that checkpoints its optimizer should checkpoint it too (opt-in; without it the first calls
after a restart simply start from a zero residual).

The reference has no such state; its nearest relatives are the config snapshots
(scripts/manage_snapshots.sh:132-143) and the never-implemented -S / -R flags
(run_codes/benchmark-core/src/utils.c:374-382)."""
from __future__ import annotations

import os

import torch

FORMAT = "ccb-residual v1"


def save_residual(path: str, residual: torch.Tensor, *, rank: int, nranks: int, codec: str, algo: str = "auto") -> None:
    """Writes one rank's fp32 residual with what is needed to refuse a wrong reload.
    The file appears atomically (written beside, then renamed)."""
    if residual.dtype != torch.float32:
        raise ValueError("the residual is kept in float32")
    blob = {"format": FORMAT, "rank": int(rank), "nranks": int(nranks), "codec": codec, "algo": algo,
            "count": residual.numel(), "residual": residual.detach().cpu().contiguous()}
    tmp = f"{path}.tmp.{os.getpid()}"
    torch.save(blob, tmp)
    os.replace(tmp, path)


def load_residual(path: str, *, rank: int, nranks: int, count: int, codec: str, device="cpu") -> torch.Tensor:
    """Returns the residual saved for exactly this (rank, world size, element count, codec);
    anything else is an error, because a residual applied to the wrong shard or scale is
    worse than none."""
    blob = torch.load(path, map_location="cpu", weights_only=True)
    if not isinstance(blob, dict) or blob.get("format") != FORMAT:
        raise ValueError(f"{path} is not a {FORMAT} file")
    want = {"rank": rank, "nranks": nranks, "count": count, "codec": codec}
    bad = {k: (blob.get(k), v) for k, v in want.items() if blob.get(k) != v}
    if bad:
        raise ValueError(f"{path} was saved for a different job: " + ", ".join(f"{k} {a} != {b}" for k, (a, b) in bad.items()))
    return blob["residual"].to(device)
