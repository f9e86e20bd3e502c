"""The C side on a GPU: benchmark drivers as processes, bare and under the preloaded
libraries (fused interposer, perf wrapper), checked through what they print and write.
Uses two ranks when the host has two GPUs, else a communicator of one rank."""
import csv
import os
import re
import shutil
from pathlib import Path

import pytest
import torch

from ccbench_b200.launch import launch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
LIBS = ROOT / "bin" / "libs"


def _ranks():
    return 2 if torch.cuda.device_count() >= 2 else 1


def _run(tmp_path, test, args, preload=(), env=None):
    exe = ROOT / "bin" / "nccl" / test / test
    assert exe.exists(), f"{exe} is not built (python -m ccbench_b200.cli build)"
    e = {"CCB_ALLOW_SINGLE_RANK": "1", "NCCL_NVLS_ENABLE": "0"}
    e.update(env or {})
    rcs, outs = launch(_ranks(), [str(exe), *args], preload=":".join(str(LIBS / p) for p in preload), env=e, cwd=str(tmp_path),
                       timeout=240, capture=True)
    assert all(rc == 0 for rc in rcs), "\n".join(o or "" for o in outs)[-3000:]
    return outs[0]


def _metric(out, name):
    vals = [float(v) for v in re.findall(rf"^\s*{name}: ([-+0-9.eE]+|nan|inf)", out, flags=re.M)]
    assert vals, f"no {name} in:\n{out[-2000:]}"
    return vals


def test_allreduce_driver_bare_then_fused(tmp_path):
    args = ["-L", "4096,1048576,33554432", "-i", "3", "-w", "1", "-d", "float", "-p", "rank_linear", "-v", "-t", "1e30",
            "-e", "rel_l2,cos_sim"]
    bare = _run(tmp_path, "allreduce", args)
    assert max(_metric(bare, "rel_l2")) < 1e-6
    for codec, lim in (("int8", 0.02), ("fp8", 0.06), ("int4", 0.3)):
        fused = _run(tmp_path, "allreduce", args, preload=["libccb_nccl.so"], env={"CCB_CODEC": codec, "CCB_VERBOSE": "1"})
        assert "[ccb_nccl]" in fused and "using NCCL" not in fused, fused[-1500:]
        rel = _metric(fused, "rel_l2")
        assert 0 < max(rel) < lim, (codec, rel)
        assert min(_metric(fused, "cos_sim")) > 0.95


@pytest.mark.parametrize("test", ["allgather", "alltoall", "bcast", "reduce", "reducescatter", "gather", "scatter"])
def test_other_collectives_under_the_interposer(tmp_path, test):
    out = _run(tmp_path, test, ["-L", "1048576", "-i", "2", "-w", "1", "-d", "float", "-v", "-t", "1e30", "-e", "rel_l2"],
               preload=["libccb_nccl.so"], env={"CCB_CODEC": "int8"})
    assert max(_metric(out, "rel_l2")) < 0.02


def test_perf_wrapper_writes_the_csv(tmp_path):
    perf_dir = tmp_path / "perf_files"
    _run(tmp_path, "allreduce", ["-L", "1048576", "-i", "4", "-w", "1", "-d", "float"], preload=["libperfnccl.so", "libccb_nccl.so"],
         env={"PERF_OUTPUT_DIR": str(perf_dir)})
    files = sorted(perf_dir.glob("*.csv"))
    assert files, list(tmp_path.rglob("*"))
    rows = list(csv.reader(open(files[0])))
    assert rows[0][:3] == ["func_name", "timestamp_us", "call_count"]
    ar = [r for r in rows[1:] if r[0] == "ncclAllReduce"]
    assert len(ar) >= 5 and all(float(r[1]) >= 0 for r in ar)


def test_result_csv_has_the_reference_columns(tmp_path):
    out_csv = tmp_path / "result.csv"
    _run(tmp_path, "allreduce", ["-L", "65536,1048576", "-i", "2", "-w", "1", "-d", "float", "-c", "-o", str(out_csv)])
    rows = list(csv.reader(open(out_csv)))
    assert len(rows) >= 3 and "msg_size" in ",".join(rows[0]).lower().replace(" ", "_")


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="point-to-point needs two GPUs")
@pytest.mark.parametrize("test", ["allgatherv", "scatterv"])
def test_compressed_point_to_point_under_the_interposer(tmp_path, test):
    """ncclSend / ncclRecv compressed by the interposer inside ncclGroupStart/End, bytes moved
    by NCCL. The report is rank 0's: in scatterv that is the root, whose own share is a plain
    copy, so only allgatherv must show a quantisation error there."""
    args = ["-L", "1048576", "-i", "2", "-w", "1", "-d", "float", "-v", "-t", "1e30", "-e", "rel_l2"]
    plain = _run(tmp_path, test, args, preload=["libccb_nccl.so"], env={"CCB_VERBOSE": "1"})
    packed = _run(tmp_path, test, args, preload=["libccb_nccl.so"], env={"CCB_P2P_CODEC": "int8", "CCB_VERBOSE": "1"})
    assert max(_metric(plain, "rel_l2")) < 1e-6
    rel = _metric(packed, "rel_l2")
    assert max(rel) < 0.02, rel
    if test == "allgatherv":
        assert max(rel) > 0, "the receive path was not compressed"


@pytest.mark.parametrize("dtype", ["bfloat16", "half"])
def test_sixteen_bit_types_through_the_driver_and_the_interposer(tmp_path, dtype):
    """`-d bfloat16` / `-d half`: pattern fill, float64 oracle, metrics and the fused kernels."""
    # rank_product values stay well inside bfloat16's range; half overflows at 65504, so it
    # gets the linear pattern on messages short enough for the sum over the ranks to fit
    sizes, pattern = ("8192,4194304", "rank_product") if dtype == "bfloat16" else ("8192,16384", "rank_linear")
    args = ["-L", sizes, "-i", "2", "-w", "1", "-d", dtype, "-p", pattern, "-v", "-t", "1e30", "-e", "rel_l2,max_abs_err,psnr"]
    bare = _run(tmp_path, "allreduce", args)
    assert max(_metric(bare, "rel_l2")) < 5e-3          # NCCL's own 16-bit result against the float64 sum
    fused = _run(tmp_path, "allreduce", args, preload=["libccb_nccl.so"], env={"CCB_CODEC": "int8", "CCB_VERBOSE": "1"})
    assert "[ccb_nccl]" in fused and "using NCCL" not in fused, fused[-1500:]
    assert 0 < max(_metric(fused, "rel_l2")) < 0.03
    assert _metric(fused, "psnr") and _metric(fused, "max_abs_err")


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="point-to-point needs two GPUs")
@pytest.mark.parametrize("test", ["pingpong", "overlap"])
def test_point_to_point_drivers_under_the_interposer(tmp_path, test):
    """The two drivers that only send and receive: plain under the interposer (NCCL moves the
    bytes untouched), and the ping-pong again with un-grouped sends and receives compressed."""
    args = ["-L", "1048576", "-i", "3", "-w", "1", "-d", "float"]
    out = _run(tmp_path, test, args, preload=["libccb_nccl.so"], env={"CCB_VERBOSE": "1"})
    assert "Test Complete" in out or "===" in out, out[-1500:]
    if test == "pingpong":
        packed = _run(tmp_path, test, args, preload=["libccb_nccl.so"], env={"CCB_P2P_CODEC": "int8"})
        assert "Test Complete" in packed or "===" in packed, packed[-1500:]
