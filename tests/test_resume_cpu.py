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


def test_report_tables(tmp_path, capsys):
    from ccbench_b200.bench import report

    csv = tmp_path / "s.csv"
    csv.write_text("msg_size,nranks,dtype,algo,codec,time_us,algbw,busbw,ref_bw,ratio,rel_l2\n"
                   "1048576,8,bf16,auto,int8,60.0,17.3,30.3,34.6,1.9,4e-3\n"
                   "1048576,8,bf16,ring,int8,130.0,8.0,14.1,16.1,1.9,1e-2\n"
                   "1048576,8,bf16,nccl,none,57.0,18.4,32.2,36.8,1.0,3e-3\n"
                   "msg_size,nranks,dtype,algo,codec,time_us,algbw,busbw,ref_bw,ratio,rel_l2\n"
                   "268435456,8,bf16,auto,int8,494.0,543,951,1087,1.9,7e-3\n"
                   "268435456,8,bf16,nccl,none,709.0,378,663,757,1.0,2e-3\n")
    assert report.main([str(csv), "--value", "busbw"]) == 0
    out = capsys.readouterr().out
    assert "### 8 ranks, bf16, busbw" in out
    assert "| 1 MiB | 30.3 | 14.1 | 32.2 | 0.95 x |" in out
    assert "| 256 MiB | 951.0 | – | 663.0 | 1.44 x |" in out
    assert report.human(8) == "8 B" and report.human(3 << 30) == "3 GiB"
