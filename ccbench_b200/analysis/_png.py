"""Heat maps without matplotlib: a plain PNG writer (zlib + CRC from the standard library)
and a viridis-like colour ramp. Used by the draw scripts when matplotlib is not installed,
so that a headless host still gets its picture; a `<name>.legend.txt` beside the image
lists what the rows, the columns and the colour range mean (there is no text rendering)."""
from __future__ import annotations

import struct
import zlib

import numpy as np

_RAMP = np.array([[68, 1, 84], [59, 82, 139], [33, 145, 140], [94, 201, 98], [253, 231, 37]], dtype=np.float64)


def colour(values: np.ndarray, vmin: float, vmax: float) -> np.ndarray:
    """[..., 3] uint8 colours of `values`; NaN is drawn light grey."""
    span = vmax - vmin if vmax > vmin else 1.0
    x = np.clip((np.nan_to_num(values, nan=vmin) - vmin) / span, 0.0, 1.0) * (len(_RAMP) - 1)
    lo = np.minimum(x.astype(int), len(_RAMP) - 2)
    frac = (x - lo)[..., None]
    rgb = _RAMP[lo] * (1 - frac) + _RAMP[lo + 1] * frac
    rgb[np.isnan(values)] = 225
    return rgb.astype(np.uint8)


def write_png(path, rgb: np.ndarray) -> None:
    """rgb: [height, width, 3] uint8."""
    h, w, _ = rgb.shape
    raw = b"".join(b"\x00" + rgb[y].tobytes() for y in range(h))

    def chunk(kind: bytes, data: bytes) -> bytes:
        return struct.pack(">I", len(data)) + kind + data + struct.pack(">I", zlib.crc32(kind + data) & 0xFFFFFFFF)

    with open(path, "wb") as f:
        f.write(b"\x89PNG\r\n\x1a\n" + chunk(b"IHDR", struct.pack(">IIBBBBB", w, h, 8, 2, 0, 0, 0)) +
                chunk(b"IDAT", zlib.compress(raw, 6)) + chunk(b"IEND", b""))


def heatmap(path, grid: np.ndarray, rows, cols_label: str, value_label: str, cell=(6, 18)) -> None:
    """Draws `grid` [rows, columns] with `cell` = (width, height) pixels per value, a colour
    bar on the right, and writes the legend file."""
    grid = np.asarray(grid, dtype=np.float64)
    finite = grid[np.isfinite(grid)]
    vmin, vmax = (float(finite.min()), float(finite.max())) if finite.size else (0.0, 1.0)
    cw, ch = cell
    body = np.repeat(np.repeat(colour(grid, vmin, vmax), ch, axis=0), cw, axis=1)
    height = body.shape[0]
    bar = colour(np.linspace(vmax, vmin, height)[:, None].repeat(16, axis=1), vmin, vmax)
    gap = np.full((height, 8, 3), 255, dtype=np.uint8)
    write_png(path, np.concatenate([body, gap, bar], axis=1))
    with open(str(path) + ".legend.txt", "w") as f:
        f.write(f"columns: {cols_label}\ncolour: {value_label}, {vmin:.6g} (dark) .. {vmax:.6g} (bright); grey = no sample\n")
        f.write("rows, top to bottom:\n" + "\n".join(f"  {i}: {r}" for i, r in enumerate(rows)) + "\n")
