"""Resume of a sweep from its CSV and persistence of the error-feedback residual."""
import pytest
import torch

from ccbench_b200.bench import sweep
from ccbench_b200.utils import state


def test_sweep_resume_keys(tmp_path):
    csv = tmp_path / "r.csv"
    csv.write_text("msg_size,nranks,dtype,algo,codec,time_us,algbw,busbw,ref_bw,ratio,rel_l2\n"
                   "1048576,8,bf16,auto,int8,60.56,17.32,30.30,34.63,1.939,4.3e-03\n"
                   "1048576,8,bf16,nccl,none,56.88,18.44,32.26,36.87,1.000,3.6e-03\n"
                   "1048576,4,bf16,ring,int8,70.00,1,1,1,1.939,1e-02\n")
    done = sweep.done_keys(str(csv), 8, "bf16")
    assert done == {(1048576, "auto", "int8"), (1048576, "nccl", "none")}
    assert (1048576, *sweep.variant_key("int8:auto")) in done
    assert (1048576, *sweep.variant_key("nccl")) in done
    assert (1048576, *sweep.variant_key("int8:ring")) not in done
    assert sweep.variant_key("int8:twoshot:4:64") == ("twoshot:4:64", "int8")
    assert sweep.done_keys(str(tmp_path / "missing.csv"), 8, "bf16") == set()


def test_residual_roundtrip_and_refusals(tmp_path):
    ef = torch.randn(1000)
    path = str(tmp_path / "ef_rank3.pt")
    state.save_residual(path, ef, rank=3, nranks=8, codec="int8")
    back = state.load_residual(path, rank=3, nranks=8, count=1000, codec="int8")
    assert torch.equal(back, ef)
    for kw in (dict(rank=2, nranks=8, count=1000, codec="int8"), dict(rank=3, nranks=4, count=1000, codec="int8"),
               dict(rank=3, nranks=8, count=999, codec="int8"), dict(rank=3, nranks=8, count=1000, codec="fp8")):
        with pytest.raises(ValueError):
            state.load_residual(path, **kw)
    with pytest.raises(ValueError):
        state.save_residual(path, ef.half(), rank=0, nranks=1, codec="int8")
    torch.save({"x": 1}, str(tmp_path / "other.pt"))
    with pytest.raises(ValueError):
        state.load_residual(str(tmp_path / "other.pt"), rank=0, nranks=1, count=1, codec="int8")
