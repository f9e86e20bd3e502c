"""NumPy restatement of the lossless float container: exact round trip for every type,
odd sizes, special values, and the expected gain on gradient-like data."""
import numpy as np
import pytest
import torch

from ccbench_b200.ops import lossless as LL


def _bits(x: torch.Tensor) -> np.ndarray:
    if x.dtype == torch.float32:
        return x.view(torch.int32).numpy().view(np.uint32)
    return x.view(torch.int16).numpy().view(np.uint16)


CODES = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("count", [1, 511, 512, 4096, 4097, 9000])
def test_round_trip_is_bit_exact(dtype, count):
    g = torch.Generator().manual_seed(count)
    x = (torch.randn(count, generator=g) * 10.0 ** torch.randint(-6, 4, (count,), generator=g)).to(dtype)
    x[::97] = 0.0
    if count > 20:
        x[3], x[7], x[11], x[13] = float("inf"), float("-inf"), float("nan"), -0.0
    bits = _bits(x)
    buf = LL.np_encode(bits, CODES[dtype])
    assert buf.size == LL.max_bytes(CODES[dtype], count)
    assert np.array_equal(LL.np_decode(buf), bits)
    assert LL.used_bytes_np(buf) <= buf.size


def test_gradient_like_data_shrinks():
    from ccbench_b200.models.workloads import gradient_like

    for dtype, lo in ((torch.bfloat16, 1.15), (torch.float32, 1.05), (torch.float16, 1.02)):
        x = gradient_like(1 << 16, dtype, seed=0)
        buf = LL.np_encode(_bits(x), CODES[dtype])
        r = x.numel() * x.element_size() / LL.used_bytes_np(buf)
        assert r > lo, (dtype, r)
    const = torch.full((8192,), 1.5, dtype=torch.bfloat16)
    r = 8192 * 2 / LL.used_bytes_np(LL.np_encode(_bits(const), 1))
    assert r > 1.9   # no exponent planes at all


def test_ratio_tool_on_the_numpy_codec(tmp_path, capsys):
    """The ratio measurement over dataset files (the role of the reference's lossless-codec
    scripts), on the NumPy codec: smooth-exponent data compresses, the table has one row per
    (file, size) and stops at the file's size."""
    import numpy as np

    from ccbench_b200.bench import lossless_ratio as R

    rng = np.random.default_rng(0)
    (rng.standard_normal(40000).astype(np.float32) * 1e-3).tofile(tmp_path / "grad.f32")
    (1.0 + rng.random(30000)).astype(np.float16).tofile(tmp_path / "act.f16")
    rows = R.run(sorted(tmp_path.iterdir()), [65536, 1 << 20], on_gpu=False)
    assert [(r["dataset"], r["bytes"]) for r in rows] == [("act", 60000), ("grad", 65536), ("grad", 160000)]
    assert all(0.5 < r["ratio"] < 1.0 for r in rows), rows
    assert R.main([str(tmp_path), "--cpu", "--sizes", "64K"]) == 0
    assert "ratio below 1.0" in capsys.readouterr().out
