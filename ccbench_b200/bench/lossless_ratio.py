"""Compression ratio (and, on a GPU, throughput) of the lossless float codec on dataset
files, one size ladder per file.

The reference measures its lossless GPU codec with two scripts (scripts/intermediate/
test_dietgpu_compress.py: one file, ratio and timings; test_dietgpu_all.py: every
dataset category at sizes from 8 KB to 512 MB). This is both: give files (raw float32 /
`.f16` / `.bf16` by extension), or a directory written by `python -m ccbench_b200.datasets`,
or nothing for synthetic categories generated on the spot.

    python -m ccbench_b200.bench.lossless_ratio dataset/            # every *.f32 under it
    python -m ccbench_b200.bench.lossless_ratio grad.f32 --sizes 8K,1M,64M
    python -m ccbench_b200.bench.lossless_ratio --cpu                # NumPy codec, no GPU

Ratio printed = compressed bytes / raw bytes (below 1 = smaller), as the reference prints."""
from __future__ import annotations

import argparse
import sys
import tempfile
from pathlib import Path

import numpy as np

from .. import datasets as D
from ..ops import lossless as LL

DEFAULT_SIZES = "8K,16K,128K,1M,8M,32M,64M,128M,256M,512M"
_EXT = {".f32": (np.float32, 0), ".f16": (np.float16, 2), ".bf16": (np.uint16, 1)}


def _load(path: Path):
    dt, code = _EXT.get(path.suffix, (np.float32, 0))
    return np.fromfile(path, dtype=dt), code


def measure(values: np.ndarray, code: int, on_gpu: bool, iters: int = 3):
    """-> (compressed bytes, encode GB/s or None, decode GB/s or None); checks the round trip."""
    raw = values.nbytes
    if not on_gpu:
        bits = values.view({4: np.uint32, 2: np.uint16}[values.itemsize])
        buf = LL.np_encode(bits, code)
        assert np.array_equal(LL.np_decode(buf, code), bits), "round trip"
        return LL.used_bytes_np(buf), None, None
    import torch

    tdt = {0: torch.float32, 1: torch.bfloat16, 2: torch.float16}[code]
    t = torch.from_numpy(values.view(np.int16) if code == 1 else values).cuda()
    t = t.view(tdt) if code == 1 else t
    comp = LL.encode(t)
    back = LL.decode(comp, t.numel(), tdt)
    assert torch.equal(back.view(torch.int16 if t.element_size() == 2 else torch.int32),
                       t.view(torch.int16 if t.element_size() == 2 else torch.int32)), "round trip"
    used = LL.used_bytes(comp)
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
    enc = dec = 0.0
    for _ in range(iters):
        ev[0].record()
        comp = LL.encode(t)
        ev[1].record()
        LL.decode(comp, t.numel(), tdt, out=back)
        ev[2].record()
        torch.cuda.synchronize()
        enc += ev[0].elapsed_time(ev[1])
        dec += ev[1].elapsed_time(ev[2])
    return used, raw * iters / enc / 1e6, raw * iters / dec / 1e6


def run(files: list[Path], sizes: list[int], on_gpu: bool, out=sys.stdout) -> list[dict]:
    rows = []
    print(f"{'dataset':<22} {'size':<8} {'ratio':<8} {'MB out':<10} {'enc GB/s':<10} {'dec GB/s':<10}", file=out)
    for f in files:
        data, code = _load(f)
        for nbytes in sizes:
            n = min(nbytes // data.itemsize, data.size)
            if n == 0:
                continue
            used, e, d = measure(data[:n], code, on_gpu)
            row = {"dataset": f.stem, "bytes": n * data.itemsize, "compressed": used, "ratio": used / (n * data.itemsize),
                   "encode_gbs": e, "decode_gbs": d}
            rows.append(row)
            fmt = lambda v: "-" if v is None else f"{v:.1f}"
            print(f"{f.stem:<22} {D.size_label(row['bytes']):<8} {row['ratio']:<8.4f} {used / 2**20:<10.2f} {fmt(e):<10} {fmt(d):<10}",
                  file=out)
            if n == data.size:
                break  # the file has nothing larger
    return rows


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("paths", nargs="*", help="files or directories; none = synthetic categories")
    ap.add_argument("--sizes", default=DEFAULT_SIZES)
    ap.add_argument("--cpu", action="store_true", help="NumPy codec (same container), ratio only")
    ap.add_argument("--synthetic-bytes", default="16M")
    a = ap.parse_args(argv)
    sizes = [D.parse_size(s) for s in a.sizes.split(",")]
    files: list[Path] = []
    with tempfile.TemporaryDirectory() as tmp:
        if not a.paths:
            files = sorted(D.synthetic(Path(tmp), D.parse_size(a.synthetic_bytes), verbose=False).values())
        for p in map(Path, a.paths):
            files += sorted(q for q in p.rglob("*") if q.suffix in _EXT) if p.is_dir() else [p]
        if not files:
            print("no dataset files found", file=sys.stderr)
            return 1
        on_gpu = not a.cpu
        if on_gpu:
            import torch

            if not torch.cuda.is_available():
                print("no GPU: use --cpu for the NumPy codec", file=sys.stderr)
                return 1
        run(files, sizes, on_gpu)
    print("ratio below 1.0 = compression achieved; lower is better")
    return 0


if __name__ == "__main__":
    sys.exit(main())
