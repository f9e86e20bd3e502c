"""The self-describing container of the error-bounded codec: pure tensor code, testable
without a GPU on a made-up buffer of group slots."""
import pytest
import torch

from ccbench_b200.ops import sz


def _fake_slots(shape, seed=0):
    ngroups = sz.capacity(shape) // sz.GROUP_STRIDE
    g = torch.Generator().manual_seed(seed)
    buf = torch.randint(0, 256, (ngroups, sz.GROUP_STRIDE), dtype=torch.uint8, generator=g)
    sizes = torch.randint(4, 500, (ngroups, 8), dtype=torch.int32, generator=g) * 16
    buf[:, :sz.GROUP_HEADER] = sizes.view(torch.uint8).reshape(ngroups, sz.GROUP_HEADER)
    return buf.view(-1), sizes


def test_roundtrip_keeps_exactly_the_used_bytes():
    shape = (40, 24, 100)
    buf, sizes = _fake_slots(shape)
    blob = sz.to_container(buf, shape, 1e-3)
    ngroups = sizes.shape[0]
    assert blob.numel() == sz.HEADER_BYTES + 4 * ngroups + int(sizes.sum()) + ngroups * sz.GROUP_HEADER
    back, shape2, eb = sz.from_container(blob)
    assert tuple(shape2) == shape and abs(eb - 1e-3) < 1e-9
    a, b = buf.view(ngroups, -1), back.view(ngroups, -1)
    for gi in range(ngroups):
        used = sz.GROUP_HEADER + int(sizes[gi].sum())
        assert torch.equal(a[gi, :used], b[gi, :used])
        assert int(b[gi, used:].max()) == 0


def test_damaged_containers_are_refused():
    shape = (16, 16, 64)
    buf, _ = _fake_slots(shape, 1)
    blob = sz.to_container(buf, shape, 1e-2)
    for cut in (blob[:-5], torch.cat([blob, blob[:3]])):
        with pytest.raises(ValueError):
            sz.from_container(cut)
    wrong = blob.clone()
    wrong[4] = 9   # version
    with pytest.raises(ValueError):
        sz.from_container(wrong)


def test_cpu_codec_round_trip_matches_the_restatement():
    import numpy as np

    rng = np.random.default_rng(0)
    zz, yy, xx = np.meshgrid(np.arange(20), np.arange(13), np.arange(70), indexing="ij")
    field = (np.sin(zz / 5.0) * np.cos(yy / 3.0) + 0.01 * xx + 1e-3 * rng.standard_normal(zz.shape)).astype(np.float32)
    eb = 1e-3
    blob = sz.encode_cpu(field, eb)
    recon, nbytes = sz.restate(field, eb)
    back = sz.decode_cpu(blob)
    assert back.shape == field.shape and np.array_equal(back, recon)
    assert float(np.abs(back - field).max()) <= np.float32(eb)
    ngroups = sz.capacity(field.shape) // sz.GROUP_STRIDE
    assert blob.size == sz.HEADER_BYTES + 4 * ngroups + nbytes + ngroups * sz.GROUP_HEADER
    # the tensor-side container reader accepts what the CPU encoder wrote
    buf, shape, eb2 = sz.from_container(torch.from_numpy(blob))
    assert tuple(shape) == field.shape and abs(eb2 - eb) < 1e-9
    assert np.array_equal(sz.decode_cpu(sz.to_container(buf, shape, eb2).numpy()), recon)


def test_cpu_codec_stores_unquantisable_tiles_raw():
    import numpy as np

    field = np.zeros((8, 8, 64), dtype=np.float32)
    field[:, :, :32] = np.linspace(-1, 1, 8 * 8 * 32, dtype=np.float32).reshape(8, 8, 32)
    field[3, 4, 40] = np.nan
    field[1, 1, 50] = 3e30
    blob = sz.encode_cpu(field, 1e-3)
    back = sz.decode_cpu(blob)
    assert np.array_equal(back[:, :, 32:], field[:, :, 32:], equal_nan=True)     # raw tile: bit exact
    assert float(np.abs(back[:, :, :32] - field[:, :, :32]).max()) <= np.float32(1e-3)
