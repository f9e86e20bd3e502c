"""The C benchmark core through ctypes (CPU only): argv front-end, size iterator,
patterns, oracle, metrics, binary dumps, perf tables, gendata capture, device map."""
import ctypes
import math
import os
import struct
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="session")
def core():
    from ccbench_b200.native_build import build_c_targets

    build_c_targets()
    os.environ["CCB_BUILTIN_METRICS"] = "1"
    return ctypes.CDLL(os.path.join(ROOT, "bin/libs/libccb_core.so"))


class SizeIter(ctypes.Structure):
    _fields_ = [("use_list", ctypes.c_int), ("index", ctypes.c_int), ("num_sizes", ctypes.c_int),
                ("size_list", ctypes.c_size_t * 256), ("min_size", ctypes.c_size_t), ("max_size", ctypes.c_size_t),
                ("incr", ctypes.c_int), ("incr_mode", ctypes.c_int)]


class CfgStruct(ctypes.Structure):
    _fields_ = [("min_message_size", ctypes.c_size_t), ("max_message_size", ctypes.c_size_t),
                ("message_size_incr", ctypes.c_int), ("message_size_incr_mode", ctypes.c_int),
                ("use_size_list", ctypes.c_int), ("num_sizes", ctypes.c_int), ("size_list", ctypes.c_size_t * 256),
                ("iterations", ctypes.c_int), ("warmup_iterations", ctypes.c_int), ("save_csv", ctypes.c_int),
                ("csv_path", ctypes.c_char * 512), ("save_binary", ctypes.c_int), ("bin_path", ctypes.c_char * 512),
                ("input_file", ctypes.c_char_p), ("file_format", ctypes.c_int), ("tolerance", ctypes.c_double),
                ("validate", ctypes.c_int), ("compute_metrics", ctypes.c_int), ("metrics_mask", ctypes.c_uint32),
                ("pattern_type", ctypes.c_int), ("data_type", ctypes.c_int), ("save_ref_path", ctypes.c_char * 512),
                ("ref_dir", ctypes.c_char * 512)]


def _parse(core, *args):
    core.parse_arguments.restype = CfgStruct
    argv = (ctypes.c_char_p * (len(args) + 1))(b"prog", *[a.encode() for a in args])
    return core.parse_arguments(len(args) + 1, argv)


def _sizes(core, cfg):
    it = SizeIter()
    core.size_iter_init(ctypes.byref(it), ctypes.byref(cfg))
    out, s = [], ctypes.c_size_t()
    while core.size_iter_next(ctypes.byref(it), ctypes.byref(s)):
        out.append(s.value)
    return out


def test_defaults_and_flags(core):
    c = _parse(core)
    assert (c.min_message_size, c.max_message_size, c.message_size_incr) == (1, 65536, 2)
    assert (c.iterations, c.warmup_iterations, c.data_type, c.pattern_type) == (100, 10, 2, 1)
    assert abs(c.tolerance - 1e-6) < 1e-18
    c = _parse(core, "-m", "8:8589934592:4", "-i", "7", "-w", "2", "-d", "float", "-p", "sequential", "-v", "-e",
               "mse,rel_l2", "-c", "-o", "r/x.csv", "-b", "-B", "r/AllReduce", "-S", "refs", "-t", "1e-3")
    assert c.max_message_size == 8589934592  # beyond the int range the reference is limited to
    assert c.iterations == 7 and c.warmup_iterations == 2 and c.data_type == 1 and c.pattern_type == 3
    assert c.validate == 1 and c.compute_metrics == 1 and c.save_csv == 1 and c.save_binary == 1
    assert c.csv_path == b"r/x.csv" and c.bin_path == b"r/AllReduce" and c.save_ref_path == b"refs"
    names = [core_name(core, i) for i in range(core.validation_registry_count())]
    assert c.metrics_mask == (1 << names.index("mse")) | (1 << names.index("rel_l2"))


def core_name(core, i):
    core.validation_metric_name.restype = ctypes.c_char_p
    return core.validation_metric_name(i).decode()


def test_metric_registry_is_sorted_and_complete(core):
    names = [core_name(core, i) for i in range(core.validation_registry_count())]
    assert names == sorted(names)
    for n in ("cos_sim", "error_distrib", "mae", "mse", "psnr", "relative_err", "ssim", "max_abs_err", "rmse", "rel_l2"):
        assert n in names


def test_size_iterator_modes(core):
    assert _sizes(core, _parse(core, "-m", "4:64:2")) == [4, 8, 16, 32, 64]
    assert _sizes(core, _parse(core, "-m", "10:50:15", "-A")) == [10, 25, 40]
    assert _sizes(core, _parse(core, "-L", "8388608,39,1024")) == [8388608, 39, 1024]


@pytest.mark.parametrize("pattern,fn", [(0, lambda r, c, i: 1), (1, lambda r, c, i: r + i),
                                        (2, lambda r, c, i: (r + 1) * (i + 1)), (3, lambda r, c, i: r * c + i)])
def test_patterns(core, pattern, fn):
    n, rank = 17, 3
    buf = (ctypes.c_float * n)()
    core.init_buffer_pattern(buf, n, 1, pattern, rank)
    assert list(buf) == [float(fn(rank, n, i)) for i in range(n)]
    ib = (ctypes.c_int * n)()
    core.init_buffer_pattern(ib, n, 0, pattern, rank)
    assert list(ib) == [fn(rank, n, i) for i in range(n)]


def test_oracle_collectives(core):
    n, count = 4, 6
    ref = (ctypes.c_double * count)()
    core.dummy_allreduce(ref, None, 2, 1, count, n)  # rank_linear: sum_r (r + i)
    assert list(ref) == [sum(r + i for r in range(n)) for i in range(count)]
    ag = (ctypes.c_float * (count * n))()
    core.dummy_allgather(ag, None, 1, 1, count, n)
    assert list(ag) == [float(r + i) for r in range(n) for i in range(count)]
    a2a = (ctypes.c_float * (count * n))()
    core.dummy_alltoall(a2a, None, 1, 3, count, n, 2)  # sequential: rank*total + index; block 2 of every sender
    total = count * n
    assert list(a2a) == [float(s * total + 2 * count + i) for s in range(n) for i in range(count)]
    rs = (ctypes.c_float * count)()
    core.dummy_reduce_scatter(rs, None, 1, 1, count, n, 1)
    assert list(rs) == [float(sum(r + count + i for r in range(n))) for i in range(count)]
    sc = (ctypes.c_float * count)()
    core.dummy_scatter(sc, None, 1, 1, count, n, 0, 3)
    assert list(sc) == [float(0 + 3 * count + i) for i in range(count)]
    bc = (ctypes.c_float * count)()
    core.dummy_bcast(bc, None, 1, 2, count, n, 2)
    assert list(bc) == [float(3 * (i + 1)) for i in range(count)]


def test_oracle_reads_files_and_folders(core, tmp_path, monkeypatch):
    data = np.arange(64, dtype=np.float32)
    f = tmp_path / "d.f32"
    data.tofile(f)
    buf = (ctypes.c_float * 8)()
    monkeypatch.delenv("DS_TYPE", raising=False)
    monkeypatch.setenv("DS_BASE_OFFSET", "16")
    core.dummy_load_rank_data(str(f).encode(), 1, 1, buf, 32, 2, 4)  # base 16 B + rank 2 * 32 B = element 20
    assert list(buf) == list(data[20:28])
    monkeypatch.setenv("DS_PER_RANK_OFFSET", "false")
    core.dummy_load_rank_data(str(f).encode(), 1, 1, buf, 32, 2, 4)
    assert list(buf) == list(data[4:12])
    monkeypatch.setenv("DS_CUSTOM_OFFSETS", "0,8,248")
    core.dummy_load_rank_data(str(f).encode(), 1, 1, buf, 32, 2, 4)  # 248 B = element 62, then zero padding
    assert list(buf) == [62.0, 63.0, 0, 0, 0, 0, 0, 0]
    monkeypatch.delenv("DS_CUSTOM_OFFSETS")
    folder = tmp_path / "dump"
    folder.mkdir()
    (data[:8] * 2).tofile(folder / "rank_1.bin")
    monkeypatch.setenv("DS_TYPE", "folder")
    core.dummy_load_rank_data(str(folder).encode(), 1, 1, buf, 32, 1, 4)
    assert list(buf) == list(data[:8] * 2)


def test_metrics_against_numpy(core, tmp_path, monkeypatch):
    rng = np.random.default_rng(0)
    ref = rng.standard_normal(1000).astype(np.float32)
    usr = (ref + 0.01 * rng.standard_normal(1000)).astype(np.float32)
    d = usr.astype(np.float64) - ref.astype(np.float64)

    def call(name):
        fn = getattr(core, f"compute_{name}")
        fn.restype = ctypes.c_double
        return fn(usr.ctypes.data_as(ctypes.c_void_p), ref.ctypes.data_as(ctypes.c_void_p), 1000, 1)

    assert math.isclose(call("mse"), np.mean(d * d), rel_tol=1e-12)
    assert math.isclose(call("rmse"), math.sqrt(np.mean(d * d)), rel_tol=1e-12)
    assert math.isclose(call("mae"), np.mean(np.abs(d)), rel_tol=1e-12)
    assert math.isclose(call("max_abs_err"), np.max(np.abs(d)), rel_tol=1e-12)
    assert math.isclose(call("rel_l2"), np.linalg.norm(d) / np.linalg.norm(ref.astype(np.float64)), rel_tol=1e-12)
    assert math.isclose(call("cos_sim"), np.dot(usr.astype(np.float64), ref) / (np.linalg.norm(usr.astype(np.float64)) * np.linalg.norm(ref.astype(np.float64))), rel_tol=1e-12)
    assert math.isclose(call("psnr"), -10 * math.log10(np.mean(d * d)), rel_tol=1e-12)
    monkeypatch.setenv("METRIC_PSNR_MAX_VAL", "10")
    assert math.isclose(call("psnr"), 20 - 10 * math.log10(np.mean(d * d)), rel_tol=1e-12)
    rel = np.mean(np.abs(d) / np.maximum(np.abs(ref.astype(np.float64)), 1e-8))
    assert math.isclose(call("relative_err"), rel, rel_tol=1e-9)
    out = tmp_path / "dist.txt"
    monkeypatch.setenv("METRIC_ERROR_DISTRIB_OUTPUT", str(out))
    p50 = call("error_distrib")
    err = np.sort(np.abs(d).astype(np.float32))
    assert math.isclose(p50, float(err[int(0.5 * 999)]), rel_tol=1e-6)
    line = out.read_text()
    assert "P99.9=" in line and "msg_bytes=4000" in line
    assert 0.99 < call("ssim") <= 1.0


def test_validate_result_and_tolerance(core):
    class Result(ctypes.Structure):
        _fields_ = [("correct", ctypes.c_int), ("num_elements", ctypes.c_size_t), ("values", ctypes.c_double * 30)]

    core.validate_result.restype = Result
    a = np.array([1.0, 2.0, 3.0], dtype=np.float32)
    b = np.array([1.0, 2.0, 3.1], dtype=np.float32)
    core.parse_metric_mask.restype = ctypes.c_uint32
    mask = core.parse_metric_mask(b"max_abs_err")
    r = core.validate_result(a.ctypes.data_as(ctypes.c_void_p), b.ctypes.data_as(ctypes.c_void_p), 3, 1, ctypes.c_double(0.05), mask)
    assert r.correct == 0 and r.num_elements == 3
    names = [core_name(core, i) for i in range(core.validation_registry_count())]
    assert abs(r.values[names.index("max_abs_err")] - 0.1) < 1e-6
    r = core.validate_result(a.ctypes.data_as(ctypes.c_void_p), b.ctypes.data_as(ctypes.c_void_p), 3, 1, ctypes.c_double(0.2), 0)
    assert r.correct == 1


def test_binary_dumps(core, tmp_path):
    base = str(tmp_path / "AllReduce").encode()
    chunk = np.arange(4, dtype=np.float32)
    for rank in range(3):
        data = (chunk + 10 * rank).astype(np.float32)
        core.write_binary_multi(base, b"user", data.ctypes.data_as(ctypes.c_void_p), ctypes.c_size_t(16), rank, 3)
    got = np.fromfile(tmp_path / "AllReduce_user.bin", dtype=np.float32)
    assert list(got) == [0, 1, 2, 3, 10, 11, 12, 13, 20, 21, 22, 23]
    core.write_binary_single(base, b"reference", chunk.ctypes.data_as(ctypes.c_void_p), ctypes.c_size_t(16), 1, 0)
    assert not (tmp_path / "AllReduce_reference.bin").exists()  # not the writer
    core.write_binary_single(base, b"reference", chunk.ctypes.data_as(ctypes.c_void_p), ctypes.c_size_t(16), 0, 0)
    assert (tmp_path / "AllReduce_reference.bin").stat().st_size == 16
    acc = np.zeros(4, dtype=np.float32)
    for _ in range(5):
        core.binary_accumulate(acc.ctypes.data_as(ctypes.c_void_p), chunk.ctypes.data_as(ctypes.c_void_p), 4, 1)
    core.binary_average(acc.ctypes.data_as(ctypes.c_void_p), 4, 1, 5)
    assert list(acc) == list(chunk)


PERF_STATE_BYTES = 1 << 21


def test_perf_table_csv_format(core, tmp_path, monkeypatch):
    class Attr(ctypes.Structure):
        _fields_ = [("key", ctypes.c_char_p), ("value", ctypes.c_double)]

    st = ctypes.create_string_buffer(PERF_STATE_BYTES)
    core.perf_init(st)
    core.perf_get_time.restype = ctypes.c_double
    t0 = core.perf_get_time()
    core.perf_notedown.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_double, ctypes.c_int, ctypes.POINTER(Attr)]
    a = (Attr * 2)(Attr(b"duration", 0.5), Attr(b"msg_bytes", 1024.0))
    core.perf_notedown(st, b"MPI_Send", t0, 2, a)
    b = (Attr * 2)(Attr(b"duration", 0.25), Attr(b"intra", 1.0))   # a column that appears later
    core.perf_notedown(st, b"MPI_Send", t0 + 1e-3, 2, b)
    c = (Attr * 1)(Attr(b"data_bytes", 64.0),)
    core.perf_notedown(st, b"MPI_Allreduce", t0 + 2e-3, 1, c)
    monkeypatch.setenv("PERF_OUTPUT_DIR", str(tmp_path / "pf"))
    assert core.perf_flush_to_rank_file(st, 3, b"perf_function") == 0
    lines = (tmp_path / "pf" / "perf_function_3.csv").read_text().splitlines()
    assert lines[0] == "func_name,timestamp_us,call_count,duration,msg_bytes,intra,data_bytes"
    f = lines[1].split(",")
    assert f[0] == "MPI_Send" and f[2] == "1.000000" and f[3] == "0.500000" and f[4] == "1024.000000" and f[5] == "" and f[6] == ""
    f = lines[2].split(",")
    assert f[2] == "2.000000" and f[4] == "" and f[5] == "1.000000"
    assert 900 < float(f[1]) - float(lines[1].split(",")[1]) < 1100  # timestamps are microseconds
    f = lines[3].split(",")
    assert f[0] == "MPI_Allreduce" and f[3] == "" and f[6] == "64.000000"
    core.perf_destroy(st)


def test_gendata_capture_dumps_and_exits(tmp_path):
    """Runs in a child process: when every target has been captured the helper flushes,
    marks done, waits for its peers (here: itself) and leaves with _exit(0)."""
    code = f"""
import ctypes, os
core = ctypes.CDLL({os.path.join(ROOT, 'bin/libs/libccb_core.so')!r})
st = ctypes.create_string_buffer({PERF_STATE_BYTES})
core.perf_init(st)
buf = bytes(range(16))
for i in range(5):
    core.perf_gendata_dump_if_target(st, b"MPI_Allreduce", buf, 16)
    core.perf_gendata_dump_if_target(st, b"MPI_Bcast", buf, 16)
print("still here")
"""
    env = dict(os.environ, PERF_GENDATA_TARGETS="allreduce:2,4;bcast:1", PERF_GENDATA_OUTPUT_DIR=str(tmp_path / "g"),
               PERF_GENDATA_DONE_DIR=str(tmp_path / "sig"), PERF_OUTPUT_DIR=str(tmp_path / "pf"), OMPI_COMM_WORLD_RANK="0",
               OMPI_COMM_WORLD_SIZE="1")
    p = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=60)
    assert p.returncode == 0 and "still here" not in p.stdout  # left early, on purpose
    assert (tmp_path / "g" / "MPI_Allreduce_000002" / "rank_0.bin").read_bytes() == bytes(range(16))
    assert (tmp_path / "g" / "MPI_Allreduce_000004" / "rank_0.bin").exists()
    assert (tmp_path / "g" / "MPI_Bcast_000001" / "rank_0.bin").exists()
    assert not (tmp_path / "g" / "MPI_Allreduce_000001").exists()
    assert (tmp_path / "sig" / "gendata_done_0").exists()
    assert (tmp_path / "pf" / "perf_function_0.csv").exists()


def test_device_map_csv(tmp_path, monkeypatch):
    from ccbench_b200 import native_build_mapper as nm

    lib = ctypes.CDLL(str(nm.build()))
    monkeypatch.setenv("PERF_OUTPUT_DIR", str(tmp_path))
    ctx = ctypes.create_string_buffer(4096 * 96 + 64)
    for rank in (1, 0):
        lib.device_map_init(ctx, rank, 2)
        lib.device_map_add_entry(ctx, b"gpu", rank)
        lib.device_map_flush_to_file(ctx)
    rows = (tmp_path / "map.csv").read_text().splitlines()
    assert rows[0] == "rank,node,device_type,device_number"
    assert {r.split(",")[0] + r.split(",")[2] + r.split(",")[3] for r in rows[1:]} == {"1gpu1", "0gpu0"}
    lib.device_map_init(ctx, 0, 1)
    lib.map_job_to_device(ctx)  # dispatcher: cpu mapper adds the affinity set
    assert struct.unpack_from("i", ctx.raw, 8 + 4096 * 88)[0] >= 0


# ------------------------------------------------------------ 16-bit float types --
# helper library: the header's inline conversions made callable
_HALF_SRC = r'''
#include "utils.h"
unsigned short t_f2bf(float f) { return ccb_float_to_bf16(f); }
float t_bf2f(unsigned short h) { return ccb_bf16_to_float(h); }
unsigned short t_f2h(float f) { return ccb_float_to_half(f); }
float t_h2f(unsigned short h) { return ccb_half_to_float(h); }
'''


@pytest.fixture(scope="session")
def halfconv(tmp_path_factory):
    d = tmp_path_factory.mktemp("half")
    (d / "h.c").write_text(_HALF_SRC)
    so = d / "libhalf.so"
    subprocess.run(["gcc", "-shared", "-fPIC", "-O2", f"-I{ROOT}/include/ccb/compat", str(d / "h.c"), "-o", str(so)], check=True)
    L = ctypes.CDLL(str(so))
    for f, a, r in (("t_f2bf", ctypes.c_float, ctypes.c_ushort), ("t_bf2f", ctypes.c_ushort, ctypes.c_float),
                    ("t_f2h", ctypes.c_float, ctypes.c_ushort), ("t_h2f", ctypes.c_ushort, ctypes.c_float)):
        getattr(L, f).argtypes, getattr(L, f).restype = [a], r
    return L


def test_half_and_bfloat16_conversions_match_numpy_and_torch(halfconv):
    import torch

    rng = np.random.default_rng(0)
    vals = np.concatenate([rng.standard_normal(2000).astype(np.float32) * 10.0 ** rng.integers(-9, 6, 2000),
                           np.array([0.0, -0.0, 1.0, 65504.0, 65520.0, 65519.9, 6e-8, 2.98e-8, 5.96e-8, 6.1e-5, 6.0e-5, 1e-10,
                                     np.inf, -np.inf, 1.0009765625, 1.00048828125, 1.001464843750], dtype=np.float32)])
    want_h = vals.astype(np.float16).view(np.uint16)
    want_b = torch.from_numpy(vals).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    for v, wh, wb in zip(vals, want_h, want_b):
        assert halfconv.t_f2h(float(v)) == int(wh), (float(v), hex(halfconv.t_f2h(float(v))), hex(int(wh)))
        assert halfconv.t_f2bf(float(v)) == int(wb), float(v)
    for bits in list(range(0, 0x10000, 37)) + [0x7c00, 0xfc00, 0x0001, 0x03ff, 0x0400, 0x8001]:
        a = halfconv.t_h2f(bits)
        b = float(np.array([bits], dtype=np.uint16).view(np.float16)[0])
        assert (math.isnan(a) and math.isnan(b)) or a == b, hex(bits)
        c = halfconv.t_bf2f(bits)
        d = float(torch.tensor([bits], dtype=torch.uint16).view(torch.bfloat16).float()[0])
        assert (math.isnan(c) and math.isnan(d)) or c == d, hex(bits)
    assert halfconv.t_f2h(float("nan")) & 0x7c00 == 0x7c00 and halfconv.t_f2h(float("nan")) & 0x3ff
    assert halfconv.t_f2bf(float("nan")) & 0x7f80 == 0x7f80 and halfconv.t_f2bf(float("nan")) & 0x7f


@pytest.mark.parametrize("name,code,npconv", [("bfloat16", 4, None), ("half", 5, np.float16)])
def test_sixteen_bit_types_through_the_core(core, name, code, npconv):
    import torch

    c = _parse(core, "-d", name)
    assert c.data_type == code
    assert _parse(core, "-d", "bf16").data_type == 4 and _parse(core, "-d", "fp16").data_type == 5
    core.get_element_size.restype = ctypes.c_size_t
    assert core.get_element_size(code) == 2
    n = 300
    buf = (ctypes.c_uint16 * n)()
    core.init_buffer_pattern(buf, n, code, 2, 3)  # rank_product, rank 3: 4 * (i + 1)
    core.to_double.restype = ctypes.c_double
    core.to_double.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int]
    got = np.array([core.to_double(buf, code, i) for i in range(n)])
    exact = torch.arange(1, n + 1, dtype=torch.float32) * 4
    want = exact.to(torch.bfloat16 if code == 4 else torch.float16).double().numpy()
    assert np.array_equal(got, want)
    # the all-reduce oracle of a 16-bit type sums in float64 and rounds once
    ref = (ctypes.c_uint16 * n)()
    core.dummy_allreduce(ref, None, code, 1, n, 4)  # rank_linear on 4 ranks: sum_r (r + i)
    ranks = [torch.arange(n, dtype=torch.float32) + r for r in range(4)]
    tdt = torch.bfloat16 if code == 4 else torch.float16
    want = sum(x.to(tdt).double() for x in ranks).to(tdt).double().numpy()
    got = np.array([core.to_double(ref, code, i) for i in range(n)])
    assert np.array_equal(got, want)
    # metrics and the tolerance compare see the converted values
    core.buffers_equal.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_double]
    other = (ctypes.c_uint16 * n)(*list(ref))
    other[5] = other[5] + 1   # one ulp off
    assert core.buffers_equal(ref, ref, n, code, 0.0) == 1
    assert core.buffers_equal(ref, other, n, code, 0.0) == 0
    assert core.buffers_equal(ref, other, n, code, 1.0) == 1
    core.compute_max_abs_err.restype = ctypes.c_double
    core.compute_max_abs_err.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int]
    err = core.compute_max_abs_err(other, ref, n, code)
    assert 0 < err <= 1.0


def test_fast_division_by_a_magic_number_is_exact_in_its_stated_range(tmp_path):
    """The multiplication that replaces run-time integer divisions in the kernels
    (csrc/kernels/ccb_fastdiv.h): every numerator below 2^22 for a spread of divisors below
    2^18, and the refusal outside that range."""
    import shutil
    import subprocess

    if not shutil.which("gcc"):
        pytest.skip("no C compiler")
    src = tmp_path / "t.c"
    src.write_text(r'''
#include <stdio.h>
#include "ccb_fastdiv.h"
int main(void) {
    unsigned long long bad = 0, n_checked = 0;
    for (unsigned d = 1; d < (1u << 18); d = d < 70 ? d + 1 : d * 3 / 2 + 1) {
        const uint64_t m = ccb_fastdiv_magic((1u << 22) - 1, d);
        if (!m) { bad++; continue; }
        for (uint32_t n = 0; n < (1u << 22); ++n) { n_checked++; if (ccb_fastdiv(n, m) != n / d) bad++; }
    }
    if (ccb_fastdiv_magic(1u << 22, 3) || ccb_fastdiv_magic(100, 1u << 18) || ccb_fastdiv_magic(100, 0)) bad++;
    printf("%llu %llu\n", n_checked, bad);
    return bad != 0;
}''')
    exe = tmp_path / "t"
    subprocess.run(["gcc", "-O2", "-I" + os.path.join(ROOT, "csrc", "kernels"), str(src), "-o", str(exe)], check=True)
    out = subprocess.run([str(exe)], capture_output=True, text=True)
    assert out.returncode == 0, out.stdout
    assert int(out.stdout.split()[0]) > 100_000_000
