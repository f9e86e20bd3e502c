"""Dataset files for the benchmarks' data-source option (DS_TYPE=file / folder).

Two ways to make them:

* from captures: tensors a training run saved per collective (`.pt`, `.npy`, raw `.bin`
  / `.f32`) are grouped into categories by file name, concatenated, tiled to a target
  size and written as raw little-endian fp32 under `<out>/<category>/`. File names and
  categories are the ones the reference's generators use
  (scripts/intermediate/generate_iter_datasets.py:29-99 writes 512 MB files,
  generate_4gb_datasets.py 4 GB ones): `activation/act_cache_512mb.f32`,
  `bwd_grad/bwd_grad_512mb.f32`, `weight/weight_512mb.f32`, `dp_grad/dp_grad_512mb.f32`,
  so run configurations written against those paths keep working.
* synthetic: when no capture exists, the same files are produced from the seeded
  generators of `models.workloads` (activations ~ normal, gradients ~ heavy-tailed,
  weights ~ normal * 0.02), which is what the headline benchmarks use.

    python -m ccbench_b200.datasets --src ~/run/datasets/iter/rank_0 --out dataset --size 512mb
    python -m ccbench_b200.datasets --synthetic --out dataset --size 64mb
"""
from __future__ import annotations

import argparse
import fnmatch
import os
import re
from pathlib import Path

import numpy as np

# category -> (output stem, file-name patterns of the captures that feed it)
CATEGORIES = {
    "activation": ("act_cache", ["SP_ReduceScatter_fwd_activation*", "PP_Comm_send_fwd_activation*", "*activation*"]),
    "bwd_grad": ("bwd_grad", ["PP_Comm_recv_bwd_grad*", "SP_AllGather_bwd_grad*", "*bwd_grad*"]),
    "weight": ("weight", ["DP_AllGather_Input_weight_shard_*", "*weight*"]),
    "dp_grad": ("dp_grad", ["DP_ReduceScatter_grad_shard_*", "*grad_shard*"]),
}
_SUFFIXES = (".pt", ".npy", ".bin", ".f32")


def parse_size(text: str) -> int:
    m = re.fullmatch(r"\s*(\d+(?:\.\d+)?)\s*([kmg]?)i?b?\s*", text.lower())
    if not m:
        raise ValueError(f"cannot read a size from {text!r}")
    return int(float(m.group(1)) * {"": 1, "k": 1 << 10, "m": 1 << 20, "g": 1 << 30}[m.group(2)])


def size_label(nbytes: int) -> str:
    for unit, name in ((1 << 30, "gb"), (1 << 20, "mb"), (1 << 10, "kb")):
        if nbytes % unit == 0:
            return f"{nbytes // unit}{name}"
    return f"{nbytes}b"


def load_flat_f32(path: Path) -> np.ndarray:
    """One capture as a flat fp32 array. A `.pt` holding a dict yields its first tensor."""
    path = Path(path)
    if path.suffix == ".pt":
        import torch

        obj = torch.load(path, map_location="cpu", weights_only=True)
        if isinstance(obj, dict):
            obj = next(v for v in obj.values() if hasattr(v, "shape"))
        elif isinstance(obj, (list, tuple)):
            obj = next(v for v in obj if hasattr(v, "shape"))
        return obj.detach().float().reshape(-1).numpy()
    if path.suffix == ".npy":
        return np.load(path).astype(np.float32, copy=False).reshape(-1)
    return np.fromfile(path, dtype="<f4")


def tile_to(arr: np.ndarray, elems: int) -> np.ndarray:
    if arr.size == 0:
        raise ValueError("cannot tile an empty capture")
    reps = -(-elems // arr.size)
    return np.tile(arr, reps)[:elems] if reps > 1 else arr[:elems]


def find_captures(src: Path, patterns) -> list[Path]:
    names = sorted(p for p in os.listdir(src) if p.endswith(_SUFFIXES))
    hit: list[str] = []
    for pat in patterns:   # earlier patterns are the specific ones; later ones only add what is new
        hit += [n for n in names if fnmatch.fnmatch(n, pat) and n not in hit]
    return [src / n for n in hit]


def write_category(out_root: Path, category: str, data: np.ndarray, nbytes: int) -> Path:
    stem = CATEGORIES[category][0]
    d = out_root / category
    d.mkdir(parents=True, exist_ok=True)
    path = d / f"{stem}_{size_label(nbytes)}.f32"
    tile_to(data.astype("<f4", copy=False), nbytes // 4).tofile(path)
    return path


def from_captures(src: Path, out_root: Path, nbytes: int, verbose: bool = True) -> dict[str, Path]:
    made = {}
    for cat, (_, pats) in CATEGORIES.items():
        files = find_captures(src, pats)
        if not files:
            if verbose:
                print(f"[{cat}] no captures under {src}, skipped")
            continue
        data = np.concatenate([load_flat_f32(f) for f in files])
        made[cat] = write_category(out_root, cat, data, nbytes)
        if verbose:
            print(f"[{cat}] {len(files)} captures, {data.size} values -> {made[cat]}")
    return made


def synthetic(out_root: Path, nbytes: int, seed: int = 0, verbose: bool = True) -> dict[str, Path]:
    import torch

    from .models.workloads import gradient_like, normal

    base = min(nbytes // 4, 16 << 20)   # 64 MB of distinct values, tiled beyond that
    gens = {
        "activation": lambda: normal(base, seed=seed).numpy(),
        "bwd_grad": lambda: gradient_like(base, torch.float32, seed=seed + 1).numpy(),
        "weight": lambda: (normal(base, seed=seed + 2) * 0.02).numpy(),
        "dp_grad": lambda: gradient_like(base, torch.float32, seed=seed + 3).numpy(),
    }
    made = {}
    for cat, g in gens.items():
        made[cat] = write_category(out_root, cat, g(), nbytes)
        if verbose:
            print(f"[{cat}] synthetic -> {made[cat]}")
    return made


def per_rank_folder(src_file: Path, out_dir: Path, nranks: int, nbytes: int) -> list[Path]:
    """Cuts one dataset file into the rank_<r>.bin files the folder data source reads
    (DS_TYPE=folder): rank r gets the r-th window of `nbytes`, wrapping around."""
    data = np.fromfile(src_file, dtype="<f4")
    out_dir.mkdir(parents=True, exist_ok=True)
    n = nbytes // 4
    paths = []
    for r in range(nranks):
        idx = (np.arange(n, dtype=np.int64) + r * n) % data.size
        p = out_dir / f"rank_{r}.bin"
        data[idx].tofile(p)
        paths.append(p)
    return paths


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="make dataset files for the benchmarks' data-source option")
    ap.add_argument("--src", default="", help="directory of captured tensors (rank_0 of a capture run)")
    ap.add_argument("--synthetic", action="store_true", help="generate instead of reading captures")
    ap.add_argument("--out", default="dataset")
    ap.add_argument("--size", default="512mb", help="bytes per output file, e.g. 512mb, 4gb")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--split", default="", help="dataset file to cut into rank_<r>.bin files")
    ap.add_argument("--ranks", type=int, default=8)
    a = ap.parse_args(argv)
    nbytes = parse_size(a.size)
    out = Path(a.out)
    if a.split:
        for p in per_rank_folder(Path(a.split), out, a.ranks, nbytes):
            print(p)
        return 0
    if a.synthetic or not a.src:
        synthetic(out, nbytes, a.seed)
        return 0
    made = from_captures(Path(os.path.expanduser(a.src)), out, nbytes)
    return 0 if made else 1


if __name__ == "__main__":
    raise SystemExit(main())
