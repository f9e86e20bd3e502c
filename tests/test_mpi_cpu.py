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


# ------------------------------------------------------------------ ZCCL-side symbol sets --
FAKE_ZCCL = r'''
/* Stand-in for libZCCL: the eight collective entry points the wrapper dispatches to. Each
 * says that it was called, pushes the data through the codec entry points ZCCL would call
 * internally (resolved through the preload chain) and finishes with the plain collective. */
#include <mpi.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
void ZCCL_float_openmp_threadblock_arg(unsigned char *, float *, size_t *, float, size_t, int);
void ZCCL_float_single_thread_arg(unsigned char *, float *, size_t *, float, size_t, int);
void ZCCL_float_decompress_openmp_threadblock_arg(float *, size_t, float, int, unsigned char *);
void ZCCL_float_decompress_single_thread_arg(float *, size_t, float, int, unsigned char *);
void ZCCL_float_homomophic_add_single_thread(unsigned char *, size_t *, size_t, float, int, unsigned char *, unsigned char *);
static void through_codec(float *x, size_t n, float tol, int block, int mt) {
    unsigned char *c = malloc(n * 4 + n / 8 + 512);
    size_t bytes = 0;
    if (mt) ZCCL_float_openmp_threadblock_arg(c, x, &bytes, tol, n, block); else ZCCL_float_single_thread_arg(c, x, &bytes, tol, n, block);
    if (mt) ZCCL_float_decompress_openmp_threadblock_arg(x, n, tol, block, c); else ZCCL_float_decompress_single_thread_arg(x, n, tol, block, c);
    free(c);
}
#define SAY(name, mt) fprintf(stderr, "[fake-zccl] %s cr=%g tol=%g block=%d mt=%d\n", name, cr, tol, block, mt)
static int ar(const void *s, void *r, float cr, float tol, int block, MPI_Aint n, MPI_Datatype dt, MPI_Op op, MPI_Comm comm, int mt) {
    SAY("allreduce", mt);
    float *t = malloc(n * 4); memcpy(t, s, n * 4); through_codec(t, n, tol, block, mt);
    if (!mt) { /* also exercise the homomorphic add: t + 0 */
        unsigned char *a = malloc(n * 4 + n / 8 + 512), *b = malloc(n * 4 + n / 8 + 512), *o = malloc(n * 4 + n / 8 + 512);
        float *z = calloc(n, 4); size_t sa, sb, so;
        ZCCL_float_single_thread_arg(a, t, &sa, tol, n, block); ZCCL_float_single_thread_arg(b, z, &sb, tol, n, block);
        ZCCL_float_homomophic_add_single_thread(o, &so, n, tol, block, a, b);
        ZCCL_float_decompress_single_thread_arg(t, n, tol, block, o);
        free(a); free(b); free(o); free(z);
    }
    int rc = PMPI_Allreduce(t, r, (int)n, dt, op, comm); free(t); return rc;
}
int MPI_Allreduce_ZCCL_RI2_mt_oa_record(const void *s, void *r, float cr, float tol, int block, MPI_Aint n, MPI_Datatype dt, MPI_Op op, MPI_Comm c) { return ar(s, r, cr, tol, block, n, dt, op, c, 1); }
int MPI_Allreduce_ZCCL_RI2_st_oa_record(const void *s, void *r, float cr, float tol, int block, MPI_Aint n, MPI_Datatype dt, MPI_Op op, MPI_Comm c) { return ar(s, r, cr, tol, block, n, dt, op, c, 0); }
int MPI_Bcast_ZCCL_mt(void *b, float cr, float tol, int block, MPI_Aint n, MPI_Datatype dt, int root, MPI_Comm c) { SAY("bcast", 1); return PMPI_Bcast(b, (int)n, dt, root, c); }
int MPI_Bcast_ZCCL(void *b, float cr, float tol, int block, MPI_Aint n, MPI_Datatype dt, int root, MPI_Comm c) { SAY("bcast", 0); return PMPI_Bcast(b, (int)n, dt, root, c); }
int MPIR_Scatter_ZCCL_mt(const void *s, float cr, float tol, int block, MPI_Aint sc, MPI_Datatype st, void *r, MPI_Aint rc, MPI_Datatype rt, int root, MPI_Comm c) { SAY("scatter", 1); return PMPI_Scatter(s, (int)sc, st, r, (int)rc, rt, root, c); }
int MPIR_Scatter_ZCCL(const void *s, float cr, float tol, int block, MPI_Aint sc, MPI_Datatype st, void *r, MPI_Aint rc, MPI_Datatype rt, int root, MPI_Comm c) { SAY("scatter", 0); return PMPI_Scatter(s, (int)sc, st, r, (int)rc, rt, root, c); }
static int agv(const void *s, MPI_Aint sc, MPI_Datatype st, void *r, const MPI_Aint *rc, MPI_Datatype rt, MPI_Comm c, float cr, float tol, int block, int mt, unsigned char *scratch) {
    SAY("allgather", mt); if (mt && !scratch) return 1; return PMPI_Allgather(s, (int)sc, st, r, (int)rc[0], rt, c);
}
int MPIR_Allgatherv_intra_ring_RI2_mt_oa_record(const void *s, MPI_Aint sc, MPI_Datatype st, void *r, const MPI_Aint *rc, const MPI_Aint *d, MPI_Datatype rt, MPI_Comm c, unsigned char *o, float cr, float tol, int block) { (void)d; return agv(s, sc, st, r, rc, rt, c, cr, tol, block, 1, o); }
int MPIR_Allgatherv_intra_ring_RI2_st_oa_record(const void *s, MPI_Aint sc, MPI_Datatype st, void *r, const MPI_Aint *rc, const MPI_Aint *d, MPI_Datatype rt, MPI_Comm c, unsigned char *o, float cr, float tol, int block) { (void)d; return agv(s, sc, st, r, rc, rt, c, cr, tol, block, 0, o); }
'''


@pytest.fixture(scope="module")
def fake_zccl(tmp_path_factory):
    d = tmp_path_factory.mktemp("zccl")
    (d / "fake_zccl.c").write_text(FAKE_ZCCL)
    inc = [] if launch_has_real_mpi() else [f"-I{ROOT / 'csrc/minimpi'}"]
    subprocess.run(["gcc", "-shared", "-fPIC", "-w", *inc, str(d / "fake_zccl.c"), "-o", str(d / "libZCCL.so")], check=True)
    return d


def launch_has_real_mpi():
    from ccbench_b200 import native_build as nb

    return nb.have_mpi()


@pytest.mark.parametrize("codec_lib", ["libsz3_for_zccl.so", "libzfp_for_zccl.so"])
@pytest.mark.parametrize("mode", ["1", "0"])
def test_zccl_wrapper_dispatch_codec_replacement_and_perf_rows(tmp_path, fake_zccl, codec_lib, mode):
    """With a libZCCL in reach the wrapper hands the four collectives to its entry points with
    the ZCCL_* settings; the codec entry points ZCCL calls are served by the preloaded
    replacement (SZ3 / ZFP role, built-in codecs here) and timed by the ZCCL perf wrapper."""
    pre = f"{LIBS / 'libperfzccl.so'}:{LIBS / codec_lib}:{LIBS / 'libmpi_zccl_wrapper.so'}"
    env = {"LD_LIBRARY_PATH": f"{fake_zccl}:{os.environ.get('LD_LIBRARY_PATH', '')}", "ZCCL_TOL": "0.002", "ZCCL_CR": "0.01",
           "ZCCL_BLOCK": "48", "ZCCL_MODE": mode, "PERF_OUTPUT_DIR": str(tmp_path / "pf")}
    outs = {}
    for test in ("allreduce", "bcast", "scatter", "allgather"):
        outs[test] = _run(2, test, pre, ["-L", "65536", "-i", "1", "-w", "0", "-d", "float", "-v", "-t", "1e30", "-e", "max_abs_err"],
                          env={**env, "PERF_OUTPUT_DIR": str(tmp_path / "pf" / test)}, cwd=tmp_path, tag=f"z{test[:2]}{mode}")
        assert f"[fake-zccl] {test}" in outs[test] and f"tol=0.002 block=48 mt={mode}" in outs[test], outs[test][-1500:]
        assert "cr=0.01" in outs[test]
    err = float(outs["allreduce"].split("max_abs_err:")[1].split()[0])
    assert err <= 2 * (3 if mode == "0" else 1) * 0.002 * 1.01 + 1e-3   # (exact for integer-valued data under the block-float codec) each rank's data went through the codec once (twice more with the add)
    rows = (tmp_path / "pf" / "allreduce" / "perf_function_0.csv").read_text().splitlines()
    names = {r.split(",")[0] for r in rows[1:]}
    want = {"ZCCL_compress_mt", "ZCCL_decompress_mt"} if mode == "1" else {"ZCCL_compress", "ZCCL_decompress_st", "ZCCL_homoadd_st"}
    assert want <= names and "MPI_Allreduce" in names, names
    cols = rows[0].split(",")
    ratio = [float(r.split(",")[cols.index("compression_ratio")]) for r in rows[1:] if r.startswith("ZCCL_compress")]
    assert ratio and 0 < min(ratio) < 0.9    # output / input, the reference's convention for these rows


def test_zccl_wrapper_without_the_library_still_compresses_within_the_tolerance(tmp_path):
    pre = f"{LIBS / 'libperfmpi.so'}:{LIBS / 'libmpi_zccl_wrapper.so'}"
    out = _run(3, "allreduce", pre, ["-L", "262144", "-i", "1", "-w", "0", "-d", "float", "-v", "-t", "1e30", "-e", "max_abs_err"],
               env={"ZCCL_TOL": "0.004", "PERF_OUTPUT_DIR": str(tmp_path / "pf")}, cwd=tmp_path, tag="zn")
    err = float(out.split("max_abs_err:")[1].split()[0])
    assert 0 < err <= 3 * 2 * 0.004 + 1e-3
    rows = (tmp_path / "pf" / "perf_function_0.csv").read_text().splitlines()
    cols = rows[0].split(",")
    ratio = [float(r.split(",")[cols.index("compression_ratio")]) for r in rows[1:] if r.startswith("mpi_compress")]
    assert ratio and min(ratio) > 1.5
