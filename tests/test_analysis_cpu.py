"""Plots on a host without matplotlib: the fallback PNG writer and the two draw scripts."""
import struct
import zlib

import numpy as np

from ccbench_b200.analysis import _png, draw_hardware, draw_perf_function


def _decode(path):
    data = open(path, "rb").read()
    assert data[:8] == b"\x89PNG\r\n\x1a\n"
    pos, chunks = 8, {}
    while pos < len(data):
        n, kind = struct.unpack(">I4s", data[pos:pos + 8])
        body = data[pos + 8:pos + 8 + n]
        assert struct.unpack(">I", data[pos + 8 + n:pos + 12 + n])[0] == zlib.crc32(kind + body) & 0xFFFFFFFF
        chunks[kind] = chunks.get(kind, b"") + body
        pos += 12 + n
    w, h = struct.unpack(">II", chunks[b"IHDR"][:8])
    raw = zlib.decompress(chunks[b"IDAT"])
    rows = np.frombuffer(raw, dtype=np.uint8).reshape(h, 1 + 3 * w)
    assert (rows[:, 0] == 0).all()
    return rows[:, 1:].reshape(h, w, 3)


def test_png_roundtrip_and_colours(tmp_path):
    grid = np.array([[0.0, 1.0, np.nan], [0.5, 0.25, 0.75]])
    _png.heatmap(tmp_path / "h.png", grid, ["a", "b"], "x", "value", cell=(2, 3))
    img = _decode(tmp_path / "h.png")
    assert img.shape == (6, 3 * 2 + 8 + 16, 3)
    assert tuple(img[0, 0]) == (68, 1, 84) and tuple(img[0, 2]) == (253, 231, 37) and tuple(img[0, 4]) == (225, 225, 225)
    legend = (tmp_path / "h.png.legend.txt").read_text()
    assert "0: a" in legend and "1: b" in legend and "value" in legend


def test_draw_scripts_write_pictures(tmp_path):
    pf = tmp_path / "perf_files"
    pf.mkdir()
    (pf / "perf_gpu_0_nodeA.csv").write_text("timestamp_sec,gpu_util,mem_util\n0.0,10,1\n0.5,50,2\n1.0,90,3\n")
    (pf / "perf_gpu_1_nodeA.csv").write_text("timestamp_sec,gpu_util,mem_util\n0.1,20,1\n0.9,80,2\n")
    (pf / "map.csv").write_text("rank,node,device_type,device_number\n0,nodeA,gpu,0\n1,nodeA,gpu,1\n")
    assert draw_hardware.main(["--perf-dir", str(pf), "--metric", "gpu_util", "--save", str(tmp_path / "hw.png")]) == 0
    assert _decode(tmp_path / "hw.png").shape[0] >= 2
    for r in (0, 1):
        (pf / f"perf_nccl_{r}.csv").write_text("func_name,timestamp_us,call_count,duration\nncclAllReduce,10,1,0.001\nncclSend,20,1,0.0005\n")
    assert draw_perf_function.main(["--perf-dir", str(pf), "--save", str(tmp_path / "fn.png")]) == 0
    assert (tmp_path / "fn.png").exists()
