"""The MPI side on CPU ranks: drivers, interposer, codec wrappers and perf wrapper,
over the bundled single-host MPI subset (or the system MPI when present)."""
import json
import os
import subprocess
import sys

import pytest

from ccbench_b200 import launch
from ccbench_b200.native_build import BIN, ROOT, build_c_targets

LIBS = BIN / "libs"


@pytest.fixture(scope="module", autouse=True)
def built():
    build_c_targets()


def _run(n, test, preload="", args=(), env=None, cwd=None, tag="t"):
    e = {"CCB_MINIMPI_JOB": f"{tag}{os.getpid()}", "BENCH_DIR": str(ROOT), "PYTHONPATH": str(ROOT)}
    e.update(env or {})
    rcs, outs = launch.launch(n, [str(BIN / "mpi" / test / test), *args], preload, e, cwd=str(cwd), timeout=120, capture=True)
    assert not any(rcs), outs[0]
    return outs[0]


@pytest.mark.parametrize("test", ["allreduce", "allgather", "alltoall", "bcast", "reduce", "gather", "scatter", "reducescatter",
                                  "allgatherv", "scatterv"])
def test_drivers_are_exact_without_wrappers(tmp_path, test):
    out = _run(3, test, args=["-L", "4096,100000", "-i", "2", "-w", "1", "-d", "double", "-v"], cwd=tmp_path, tag=test[:4])
    assert out.count("Correct: YES") == 2 and "NO" not in out.replace("NOT", "")


@pytest.mark.parametrize("n", [2, 3, 4])
def test_interposer_with_int8_codec_stays_within_the_quantisation_error(tmp_path, n):
    pre = f"{LIBS / 'libmpi_int8.so'}:{LIBS / 'libplain_mpi_compress.so'}"
    for test in ("allreduce", "reducescatter", "allgather", "bcast", "alltoall", "reduce"):
        out = _run(n, test, pre, ["-L", "262144", "-i", "2", "-w", "1", "-d", "float", "-v", "-t", "1e30", "-e", "rel_l2,max_abs_err"],
                   cwd=tmp_path, tag=f"{test[:3]}{n}")
        rel = float(out.split("rel_l2:")[1].split()[0])
        assert rel < 0.02, (test, out)
    # pass-through switch
    out = _run(n, "allreduce", pre, ["-L", "65536", "-i", "1", "-w", "0", "-d", "float", "-v"], env={"MPI_COMPRESS_DISABLE": "1"},
               cwd=tmp_path, tag=f"dis{n}")
    assert "Correct: YES" in out


def test_error_bounded_cpu_codec_and_perf_rows(tmp_path):
    pre = f"{LIBS / 'libperfmpi.so'}:{LIBS / 'libmpi_szcpu.so'}:{LIBS / 'libplain_mpi_compress.so'}"
    out = _run(2, "allreduce", pre, ["-L", "400000", "-i", "2", "-w", "1", "-d", "float", "-v", "-t", "1e30", "-e", "max_abs_err"],
               env={"MPI_SZ3_ABS_EB": "1e-2", "PERF_OUTPUT_DIR": str(tmp_path / "pf")}, cwd=tmp_path, tag="sz")
    err = float(out.split("max_abs_err:")[1].split()[0])
    assert err <= 2 * 1e-2 * 2 + 1e-3  # one bounded hop each way plus fp32 rounding of ~1e5-sized values
    rows = (tmp_path / "pf" / "perf_function_1.csv").read_text().splitlines()
    cols = rows[0].split(",")
    assert cols[:3] == ["func_name", "timestamp_us", "call_count"] and "compression_ratio" in cols and "data_bytes" in cols
    names = {r.split(",")[0] for r in rows[1:]}
    assert {"mpi_compress", "mpi_decompress", "MPI_Allreduce"} <= names
    ratio = [float(r.split(",")[cols.index("compression_ratio")]) for r in rows[1:] if r.startswith("mpi_compress")]
    assert min(ratio) > 1.5
    assert all(float(r.split(",")[1]) >= 0 for r in rows[1:])


@pytest.mark.parametrize("rate,limit", [(16, 2e-4), (8, 5e-2)])
def test_fixed_rate_cpu_codec(tmp_path, rate, limit):
    pre = f"{LIBS / 'libperfmpi.so'}:{LIBS / 'libmpi_zfp.so'}:{LIBS / 'libplain_mpi_compress.so'}"
    out = _run(2, "allreduce", pre, ["-L", "262144", "-i", "2", "-w", "1", "-d", "float", "-v", "-t", "1e30", "-e", "rel_l2"],
               env={"MPI_ZFP_RATE": str(rate), "PERF_OUTPUT_DIR": str(tmp_path / "pf")}, cwd=tmp_path, tag=f"zf{rate}")
    rel = float(out.split("rel_l2:")[1].split()[0])
    assert 0 < rel < limit, out
    rows = (tmp_path / "pf" / "perf_function_0.csv").read_text().splitlines()
    cols = rows[0].split(",")
    ratio = [float(r.split(",")[cols.index("compression_ratio")]) for r in rows[1:] if r.startswith("mpi_compress")]
    # fixed rate: 32 bits in, `rate` bits (+ 16 per 64 values) out, whatever the data
    assert all(abs(x - 32.0 / (rate + 0.25)) < 0.05 * 32.0 / rate for x in ratio), ratio


def test_collectives_and_codec_in_one_library(tmp_path):
    pre = str(LIBS / "libmpi_zccl_wrapper.so")
    for test in ("allreduce", "bcast", "allgather", "scatter"):
        out = _run(3, test, pre, ["-L", "200000", "-i", "1", "-w", "1", "-d", "float", "-v", "-t", "1e30", "-e", "max_abs_err"],
                   env={"ZCCL_TOL": "1e-3"}, cwd=tmp_path, tag=f"zc{test[:3]}")
        err = float(out.split("max_abs_err:")[1].split()[0])
        assert err <= 3 * 1e-3 * 3 + 1e-3, (test, out)
        if test in ("allreduce", "allgather"):   # the report is rank 0's; a root keeps its own exact copy
            assert err > 0, (test, out)


def test_pingpong_csv_layout(tmp_path):
    _run(2, "pingpong", args=["-L", "1024,65536", "-i", "3", "-w", "1", "-c", "-o", str(tmp_path / "pp.csv")], cwd=tmp_path, tag="pp")
    rows = (tmp_path / "pp.csv").read_text().splitlines()
    assert rows[0] == "msg_size,partner,comm_type,latency_us,bandwidth_gbps,send0_us,recv0_us,recvP_us,sendP_us"
    assert len(rows) == 3 and rows[1].split(",")[:3] == ["1024", "1", "intra"]


def test_config1_cpu_benchmark():
    p = subprocess.run([sys.executable, "-m", "ccbench_b200.bench.config1_cpu", "--elements", "65536", "--iters", "2"], cwd=ROOT,
                       capture_output=True, text=True, timeout=300)
    assert p.returncode == 0, p.stdout + p.stderr
    res = json.loads(p.stdout)
    assert res["uncompressed"]["rel_l2"] < 1e-6
    q = res["int8_block"]
    assert 3.5 < q["compression_ratio"] < 4.0 and 1e-4 < q["rel_l2"] < 0.02 and q["max_abs_err"] < 0.1
