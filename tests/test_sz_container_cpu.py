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
