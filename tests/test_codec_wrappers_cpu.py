"""The SZ3 and ZFP compression wrappers of the MPI path: with the real library's entry points
present (stand-in libraries here, found through LD_LIBRARY_PATH exactly as a real libSZ3c.so /
libzfp.so would be) they drive the library with the values of the reference's environment
variables; without it they fall back to the built-in codecs and keep the promised bounds."""
import ctypes
import os
import subprocess
import sys
import textwrap
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
LIBS = ROOT / "bin" / "libs"

FAKE_SZ3 = r'''
#include <stdlib.h>
#include <string.h>
/* records what it was called with in front of a raw copy of the data */
unsigned char *SZ_compress_args(int type, void *data, size_t *outSize, int mode, double abs_eb, double rel_eb, double pw,
                                size_t r5, size_t r4, size_t r3, size_t r2, size_t r1) {
    (void)pw; (void)r5; (void)r4; (void)r3; (void)r2;
    const size_t bytes = r1 * (type == 1 ? 8 : 4);
    unsigned char *b = malloc(40 + bytes);
    double hdr[5] = {(double)type, (double)mode, abs_eb, rel_eb, (double)r1};
    memcpy(b, hdr, 40); memcpy(b + 40, data, bytes); *outSize = 40 + bytes; return b;
}
void *SZ_decompress(int type, unsigned char *bytes, size_t len, size_t r5, size_t r4, size_t r3, size_t r2, size_t r1) {
    (void)type; (void)r5; (void)r4; (void)r3; (void)r2; (void)r1;
    void *o = malloc(len - 40); memcpy(o, bytes + 40, len - 40); return o;
}
'''

FAKE_ZFP = r'''
#include <stdlib.h>
#include <string.h>
typedef struct { void *buf; size_t cap; } bs_t;
typedef struct { bs_t *bs; double tag[6]; } zs_t;
typedef struct { void *data; int type; size_t n; } fld_t;
void *stream_open(void *b, size_t n) { bs_t *s = malloc(sizeof *s); s->buf = b; s->cap = n; return s; }
void stream_close(void *s) { free(s); }
void *zfp_stream_open(void *bs) { zs_t *z = calloc(1, sizeof *z); z->bs = bs; return z; }
void zfp_stream_close(void *z) { free(z); }
int zfp_stream_set_params(void *z, unsigned a, unsigned b, unsigned c, int d) { double t[6] = {1, a, b, c, d, 0}; memcpy(((zs_t *)z)->tag, t, 48); return 1; }
double zfp_stream_set_rate(void *z, double r, int type, unsigned dims, int al) { double t[6] = {2, r, type, dims, al, 0}; memcpy(((zs_t *)z)->tag, t, 48); return r; }
unsigned zfp_stream_set_precision(void *z, unsigned p) { double t[6] = {3, p, 0, 0, 0, 0}; memcpy(((zs_t *)z)->tag, t, 48); return p; }
double zfp_stream_set_accuracy(void *z, double tol) { double t[6] = {4, tol, 0, 0, 0, 0}; memcpy(((zs_t *)z)->tag, t, 48); return tol; }
void zfp_stream_set_reversible(void *z) { double t[6] = {5, 0, 0, 0, 0, 0}; memcpy(((zs_t *)z)->tag, t, 48); }
void *zfp_field_1d(void *d, int type, size_t n) { fld_t *f = malloc(sizeof *f); f->data = d; f->type = type; f->n = n; return f; }
void zfp_field_free(void *f) { free(f); }
size_t zfp_compress(void *z_, const void *f_) {
    zs_t *z = z_; const fld_t *f = f_; const size_t bytes = f->n * (f->type == 4 ? 8 : 4);
    if (48 + bytes > z->bs->cap) return 0;
    memcpy(z->bs->buf, z->tag, 48); memcpy((char *)z->bs->buf + 48, f->data, bytes); return 48 + bytes;
}
size_t zfp_decompress(void *z_, void *f_) {
    zs_t *z = z_; fld_t *f = f_; const size_t bytes = f->n * (f->type == 4 ? 8 : 4);
    memcpy(f->data, (char *)z->bs->buf + 48, bytes); return 48 + bytes;
}
'''

DRIVER = textwrap.dedent('''
    import ctypes, sys, json
    import numpy as np
    lib, n, dbl = sys.argv[1], int(sys.argv[2]), sys.argv[3] == "1"
    L = ctypes.CDLL(lib)
    L.mpi_compress.argtypes = [ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p, ctypes.POINTER(ctypes.c_size_t)]
    L.mpi_decompress.argtypes = [ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p, ctypes.c_size_t]
    rng = np.random.default_rng(0)
    x = np.cumsum(rng.standard_normal(n)).astype(np.float64 if dbl else np.float32) * 0.01
    out = np.zeros(x.nbytes + 4096, dtype=np.uint8)
    size = ctypes.c_size_t(out.size)
    rc1 = L.mpi_compress(x.ctypes.data, x.nbytes, out.ctypes.data, ctypes.byref(size))
    y = np.zeros_like(x)
    rc2 = L.mpi_decompress(out.ctypes.data, size.value, y.ctypes.data, y.nbytes)
    head = out[:48].view(np.float64).tolist()
    print(json.dumps({"rc": [rc1, rc2], "size": size.value, "raw": x.nbytes, "maxerr": float(np.abs(x.astype(np.float64) - y).max()),
                      "range": float(x.max() - x.min()), "head": head}))
''')


@pytest.fixture(scope="module")
def built(tmp_path_factory):
    from ccbench_b200.native_build import build_c_targets

    build_c_targets()
    d = tmp_path_factory.mktemp("fakelibs")
    for name, src in (("libSZ3c.so", FAKE_SZ3), ("libzfp.so", FAKE_ZFP)):
        (d / (name + ".c")).write_text(src)
        subprocess.run(["gcc", "-shared", "-fPIC", str(d / (name + ".c")), "-o", str(d / name)], check=True)
    (d / "driver.py").write_text(DRIVER)
    return d


def _run(built, lib, n, env, with_fake, dbl=False):
    import json

    e = {k: v for k, v in os.environ.items() if not k.startswith(("MPI_SZ3", "MPI_ZFP"))}
    e.update(env)
    e["LD_LIBRARY_PATH"] = (str(built) + ":" if with_fake else "") + e.get("LD_LIBRARY_PATH", "")
    p = subprocess.run([sys.executable, str(built / "driver.py"), str(LIBS / lib), str(n), "1" if dbl else "0"], env=e,
                       capture_output=True, text=True, timeout=120)
    assert p.returncode == 0, p.stderr[-2000:]
    return json.loads(p.stdout.strip().splitlines()[-1]), p.stderr


def test_sz3_wrapper_drives_the_library_when_it_is_there(built):
    r, err = _run(built, "libmpi_sz3.so", 5000, {"MPI_SZ3_TYPE": "1", "MPI_SZ3_EB_MODE": "1", "MPI_SZ3_ABS_EB": "2e-5",
                                                   "MPI_SZ3_REL_EB": "0.003"}, True, dbl=True)
    assert "loaded libSZ3c.so" in err
    assert r["rc"] == [0, 0] and r["maxerr"] == 0.0
    assert r["head"][:5] == [1.0, 1.0, 2e-5, 0.003, 5000.0]   # type, mode, bounds, 1-D length
    r, _ = _run(built, "libmpi_sz3.so", 777, {}, True)
    assert r["head"][:5] == [0.0, 0.0, 1e-6, 0.01, 777.0]      # the reference's defaults


def test_sz3_wrapper_falls_back_to_the_builtin_codec(built):
    r, err = _run(built, "libmpi_sz3.so", 40000, {"MPI_SZ3_ABS_EB": "1e-3"}, False)
    assert "built-in" in err and r["rc"] == [0, 0]
    assert 0 < r["maxerr"] <= 1e-3 and r["size"] < 0.6 * r["raw"]
    r, _ = _run(built, "libmpi_sz3.so", 40000, {"MPI_SZ3_EB_MODE": "1", "MPI_SZ3_REL_EB": "1e-3"}, False)
    assert 0 < r["maxerr"] <= 1e-3 * r["range"] * 1.0001
    r, _ = _run(built, "libmpi_sz3.so", 3000, {"MPI_SZ3_FORCE_BUILTIN": "1", "MPI_SZ3_TYPE": "double", "MPI_SZ3_ABS_EB": "1e-4"},
                True, dbl=True)
    assert 0 < r["maxerr"] <= 1e-4


@pytest.mark.parametrize("env,tag", [
    ({"MPI_ZFP_MODE": "1", "MPI_ZFP_MINBITS": "3", "MPI_ZFP_MAXBITS": "900", "MPI_ZFP_MAXPREC": "12", "MPI_ZFP_MINEXP": "-9"}, [1, 3, 900, 12, -9]),
    ({}, [2, 16.0, 3, 1, 0]),
    ({"MPI_ZFP_MODE": "2", "MPI_ZFP_RATE": "9.5", "MPI_ZFP_TYPE": "4"}, [2, 9.5, 4, 1, 0]),
    ({"MPI_ZFP_MODE": "3", "MPI_ZFP_PREC": "14"}, [3, 14, 0, 0, 0]),
    ({"MPI_ZFP_MODE": "4", "MPI_ZFP_TOL": "0.25"}, [4, 0.25, 0, 0, 0]),
    ({"MPI_ZFP_MODE": "5"}, [5, 0, 0, 0, 0]),
])
def test_zfp_wrapper_configures_the_library_in_all_five_modes(built, env, tag):
    r, err = _run(built, "libmpi_zfp.so", 1000, env, True, dbl=env.get("MPI_ZFP_TYPE") == "4")
    assert "loaded libzfp.so" in err and r["rc"] == [0, 0] and r["maxerr"] == 0.0
    assert r["head"][:5] == [float(t) for t in tag]


def test_zfp_builtin_codec_modes(built):
    n = 20000
    r, err = _run(built, "libmpi_zfp.so", n, {"MPI_ZFP_RATE": "12"}, False)
    assert "built-in" in err and r["rc"] == [0, 0]
    assert r["size"] == 8 + (n + 63) // 64 * (3 + 96)           # fixed rate: the size depends on the count only
    r8, _ = _run(built, "libmpi_zfp.so", n, {"MPI_ZFP_RATE": "8"}, False)
    assert r8["maxerr"] > r["maxerr"] > 0
    acc, _ = _run(built, "libmpi_zfp.so", n, {"MPI_ZFP_MODE": "4", "MPI_ZFP_TOL": "1e-3"}, False)
    assert 0 < acc["maxerr"] <= 1e-3
    loose, _ = _run(built, "libmpi_zfp.so", n, {"MPI_ZFP_MODE": "4", "MPI_ZFP_TOL": "0.05"}, False)
    assert loose["maxerr"] <= 0.05 and loose["size"] < acc["size"]
    prec, _ = _run(built, "libmpi_zfp.so", n, {"MPI_ZFP_MODE": "3", "MPI_ZFP_PREC": "20"}, False)
    assert prec["maxerr"] < r8["maxerr"]
    exp_, _ = _run(built, "libmpi_zfp.so", n, {"MPI_ZFP_MODE": "1", "MPI_ZFP_MINEXP": "-8", "MPI_ZFP_MAXPREC": "24"}, False)
    assert 0 < exp_["maxerr"] <= 2.0 ** -8
    rev, _ = _run(built, "libmpi_zfp.so", n, {"MPI_ZFP_MODE": "5"}, False, dbl=True)
    assert rev["maxerr"] == 0.0 and rev["size"] == 8 + rev["raw"]
