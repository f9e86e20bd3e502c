"""CPU checks of the torch restatements of the codecs and algorithms."""
import torch

from ccbench_b200.ops import codecs as C


def test_int8_roundtrip_error_bound():
    x = torch.randn(10000) * 3
    d = C.int8_roundtrip(x, 128)
    xb = torch.cat([x, x.new_zeros((-x.numel()) % 128)]).reshape(-1, 128)
    bound = (xb.abs().amax(1, keepdim=True) / 254).expand_as(xb).reshape(-1)[: x.numel()]
    assert ((d - x).abs() <= bound * 1.0001 + 1e-12).all()


def test_fp8_scale_is_smallest_power_of_two():
    for m in [1e-30, 1e-3, 0.9, 1.0, 447.9, 448.0, 448.1, 1e6, 3.5e9]:
        e = C.ue8m0_exponent(torch.tensor([m])).item()
        if -126 < e < 126:
            assert m * 2.0 ** -e <= 448.0
            assert m * 2.0 ** -(e - 1) > 448.0
    x = torch.randn(4096) * 10
    d = C.fp8_roundtrip(x)
    assert ((d - x).abs() <= x.abs() * 0.0626 + 1e-3).all()  # e4m3 has 3 mantissa bits


def test_zero_block_and_padding():
    x = torch.zeros(100)
    assert C.int8_roundtrip(x).abs().sum() == 0
    assert C.fp8_roundtrip(x).abs().sum() == 0
    y = torch.randn(130)
    assert C.int8_roundtrip(y).shape == y.shape


def test_simulated_algorithms_agree_with_exact_sum():
    g = torch.Generator().manual_seed(0)
    for n in (1, 2, 3, 8):
        xs = [torch.randn(3000, generator=g) for _ in range(n)]
        exact = sum(xs)
        for algo in ("oneshot", "twoshot", "ring", "tree"):
            out = C.simulate_all_reduce(xs, "none", algo)
            assert torch.allclose(out, exact, atol=1e-5)
            out8 = C.simulate_all_reduce(xs, "int8", algo)
            assert ((out8 - exact).norm() / exact.norm()) < 0.03


def test_reference_wire_layout():
    x = torch.randn(600)
    inv, q = C.int8_encode_reference_wire(x, 256)
    assert inv.numel() == 3 and q.numel() == 600
    d = q[:256].float() / inv[0]
    assert (d - x[:256]).abs().max() <= x[:256].abs().max() / 254 * 1.001


def test_wire_bytes_of_every_codec():
    """Slot size = payload of the padded element count + its scales, rounded to 256 bytes."""
    import torch

    from ccbench_b200.comm import wire_bytes

    def want(codec, es, count):
        pad = -(-count // 512) * 512
        b = {"none": pad * es, "int8": pad + pad // 128 * 4, "int8_g256": pad + pad // 256 * 4, "fp8": pad + pad // 32,
             "int4": pad // 2 + pad // 128 * 4}[codec]
        return -(-b // 256) * 256

    for codec in ("none", "int8", "int8_g256", "fp8", "int4"):
        for dt, es in ((torch.float32, 4), (torch.bfloat16, 2)):
            for count in (1, 512, 513, 100000, (1 << 20) + 7):
                assert wire_bytes(codec, dt, count) == want(codec, es, count), (codec, dt, count)


def test_int4_restatement_properties():
    import torch

    from ccbench_b200.ops import codecs as C

    x = torch.randn(1000, generator=torch.Generator().manual_seed(0))
    y = C.roundtrip(x, "int4")
    grp = torch.cat([x, torch.zeros(24)]).view(-1, 128).abs().amax(dim=1)
    step = (grp / 7).repeat_interleave(128)[:1000]
    assert ((x - y).abs() <= 0.5 * step + 1e-7).all()
    assert torch.equal(C.roundtrip(y, "int4"), y)          # idempotent: codes survive a second trip
    assert abs(C.wire_ratio("int4", torch.bfloat16) - 2 / (0.5 + 4 / 128)) < 1e-9
