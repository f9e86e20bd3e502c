"""Stand-alone codec kernels and the reference-wire kernels against the torch restatements."""
import pytest
import torch

from ccbench_b200.ops import codecs as C
from ccbench_b200.ops import standalone as S

pytestmark = pytest.mark.gpu
DT = {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16}


@pytest.mark.parametrize("codec", ["int8", "int8_g256", "fp8", "int4", "none"])
@pytest.mark.parametrize("dt", ["f32", "bf16", "f16"])
@pytest.mark.parametrize("count", [1, 511, 4096, 100003])
def test_encode_decode_matches_the_restatement(codec, dt, count):
    dtype = DT[dt]
    x = (torch.randn(count, generator=torch.Generator().manual_seed(count)) * 3).to(dtype)
    wire = S.encode(x.cuda(), codec)
    got = S.decode(wire, codec, count, dtype).float().cpu()
    want = C.roundtrip(x.float(), codec, dtype).to(dtype).float()
    assert torch.equal(got, want)


@pytest.mark.parametrize("codec", ["int8", "fp8", "int4"])
def test_decode_reduce_and_reduce_recode(codec):
    count = 70001
    g = torch.Generator().manual_seed(7)
    xs = [torch.randn(count, generator=g) for _ in range(5)]
    wires = [S.encode(x.cuda(), codec) for x in xs]
    acc = torch.zeros(count, device="cuda")
    for w in wires:
        S.decode_reduce(w, codec, acc)
    want = sum(C.roundtrip(x, codec) for x in xs)
    assert torch.allclose(acc.cpu(), want, rtol=1e-6, atol=1e-6)
    fused = S.decode(S.reduce_recode(wires, codec, count), codec, count, torch.float32).cpu()
    step = {"int8": 1 / 127, "fp8": 1 / 8, "int4": 1 / 7}[codec]
    assert (fused - want).abs().max().item() <= 0.51 * step * want.abs().max().item() * 1.05
    torch.cuda.synchronize()


@pytest.mark.parametrize("group", [128, 256])
def test_reference_wire_layout(group):
    count = 5000
    x = torch.randn(count, generator=torch.Generator().manual_seed(3))
    wire = S.refwire_encode(x.cuda(), group).cpu()
    inv, q = C.int8_encode_reference_wire(x, group)
    ng = (count + group - 1) // group
    assert torch.equal(wire[: ng * 4].view(torch.float32), inv)
    assert torch.equal(wire[ng * 4:].view(torch.int8), q)
    back = S.refwire_decode(wire.cuda(), count, torch.float32, group).cpu()
    assert torch.allclose(back, q.float() / inv.repeat_interleave(group)[:count], rtol=1e-6, atol=0)
