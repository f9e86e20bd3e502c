"""The NCCL-free provider exports every nccl* symbol that the benchmark drivers and the
extension library import, so preloading it leaves no call for libnccl."""
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
LIB = ROOT / "bin" / "libs" / "libccb_nccl_standalone.so"


def _symbols(path, defined):
    flag = "--defined-only" if defined else "--undefined-only"
    out = subprocess.run(["nm", "-D", flag, str(path)], capture_output=True, text=True, check=True).stdout
    return {line.split()[-1].split("@")[0] for line in out.splitlines() if line.strip()}


def test_every_nccl_symbol_the_drivers_import_is_served():
    drivers = sorted((ROOT / "bin" / "nccl").glob("*/*"))
    if not LIB.exists() or not drivers:
        pytest.skip("native side not built (python -m ccbench_b200.cli build)")
    have = _symbols(LIB, True)
    assert not any(s.startswith("nccl") for s in _symbols(LIB, False)), "the provider itself must not import NCCL"
    ext = ROOT / "bin" / "libs" / "libnccl_extensions.so"
    served_by_extensions = _symbols(ext, True) if ext.exists() else set()
    missing = {}
    for exe in [*drivers, *([ext] if ext.exists() else [])]:
        if exe.is_file():
            want = {s for s in _symbols(exe, False) if s.startswith("nccl")}
            lack = want - have - served_by_extensions
            if lack:
                missing[exe.name] = sorted(lack)
    assert not missing, missing


# ---- the provider's host logic against a stand-in runtime (no GPU, no CUDA call) ----------
STUB = r"""
#include <stdint.h>
#include <stdio.h>
#include <string.h>
#include "ccb/ccb.h"
typedef struct { int kind; int a, b; unsigned long long bytes; const void *p0, *p1; } rec_t;   /* kind: 1 p2p op, 2 memcpy, 3 fused call, 4 fold */
static rec_t g_log[256];
static int g_n;
static int g_rank, g_ranks;
static void rec(int kind, int a, int b, unsigned long long bytes, const void *p0, const void *p1) {
    if (g_n < 256) g_log[g_n++] = (rec_t){kind, a, b, bytes, p0, p1};
}
int stub_count(void) { return g_n; }
void stub_get(int i, int *kind, int *a, int *b, unsigned long long *bytes) { *kind = g_log[i].kind; *a = g_log[i].a; *b = g_log[i].b; *bytes = g_log[i].bytes; }
void stub_reset(void) { g_n = 0; }
/* libccb */
int ccb_comm_create(ccb_comm **out, int rank, int nranks, const char *tag, uint64_t arena, int flags) {
    (void)arena; (void)flags;
    if (strlen(tag) != 33 || tag[0] != 's') return CCB_ERR_ARG;
    g_rank = rank; g_ranks = nranks; *out = (ccb_comm *)&g_rank; return CCB_OK;
}
int ccb_comm_destroy(ccb_comm *c) { (void)c; return CCB_OK; }
int ccb_comm_status(ccb_comm *c, uint32_t *w) { (void)c; memset(w, 0, 32); return CCB_OK; }
const char *ccb_last_error(void) { return "stub"; }
uint64_t ccb_launch_count(void) { return 0; }
int ccb_p2p(ccb_comm *c, const ccb_p2p_op *ops, int n, ccb_stream_t s) {
    (void)c; (void)s;
    for (int i = 0; i < n; ++i) rec(1, ops[i].peer, ops[i].is_recv, ops[i].bytes, ops[i].buf, NULL);
    return CCB_OK;
}
int ccb_fold(int xt, int op, const void *parts, uint64_t stride, int np, uint64_t count, void *out, ccb_stream_t s) {
    (void)stride; (void)s; rec(4, xt, op * 100 + np, count, parts, out); return CCB_OK;
}
#define FUSED(name, id) int name
int ccb_all_reduce(ccb_comm *c, const void *const *s, void *const *r, uint64_t count, int dt, int op, int codec, int algo, float *const *ef, ccb_stream_t st) {
    (void)c; (void)algo; (void)ef; (void)st; rec(3, dt, op * 100 + codec, count, s[0], r[0]);
    return count > (1u << 20) ? CCB_ERR_CAPACITY : CCB_OK;   /* large calls must be cut into pieces */
}
int ccb_reduce_scatter(ccb_comm *c, const void *const *s, void *const *r, uint64_t count, int dt, int op, int codec, float *const *ef, ccb_stream_t st) {
    (void)c; (void)ef; (void)st; rec(3, dt, 1000 + op * 100 + codec, count, s[0], r[0]); return CCB_OK; }
int ccb_reduce(ccb_comm *c, const void *const *s, void *const *r, uint64_t count, int dt, int op, int root, int codec, ccb_stream_t st) {
    (void)c; (void)st; (void)codec; rec(3, dt, 2000 + root, count, s[0], r[0]); return CCB_OK; }
int ccb_all_gather(ccb_comm *c, const void *const *s, void *const *r, uint64_t count, int dt, int codec, ccb_stream_t st) {
    (void)c; (void)st; (void)codec; rec(3, dt, 3000, count, s[0], r[0]); return CCB_OK; }
int ccb_broadcast(ccb_comm *c, const void *const *s, void *const *r, uint64_t count, int dt, int root, int codec, ccb_stream_t st) {
    (void)c; (void)st; (void)codec; rec(3, dt, 4000 + root, count, s[0], r[0]); return CCB_OK; }
int ccb_all_to_all(ccb_comm *c, const void *const *s, void *const *r, uint64_t count, int dt, int codec, ccb_stream_t st) {
    (void)c; (void)st; (void)codec; rec(3, dt, 5000, count, s[0], r[0]); return CCB_OK; }
/* CUDA runtime */
typedef int cudaError_t; typedef void *cudaStream_t;
cudaError_t cudaGetDevice(int *d) { *d = 0; return 0; }
cudaError_t cudaSetDevice(int d) { (void)d; return 0; }
cudaError_t cudaMemcpyAsync(void *d, const void *s, size_t n, int kind, cudaStream_t st) { (void)kind; (void)st; rec(2, 0, 0, n, s, d); return 0; }
static char g_pool[1 << 16];
cudaError_t cudaMallocAsync(void **p, size_t n, cudaStream_t st) { (void)n; (void)st; *p = g_pool; return 0; }
cudaError_t cudaFreeAsync(void *p, cudaStream_t st) { (void)p; (void)st; return 0; }
cudaError_t cudaMalloc(void **p, size_t n) { (void)n; *p = g_pool; return 0; }
cudaError_t cudaFree(void *p) { (void)p; return 0; }
"""


@pytest.fixture(scope="module")
def provider(tmp_path_factory):
    import ctypes
    import shutil

    if not shutil.which("gcc"):
        pytest.skip("no C compiler")
    d = tmp_path_factory.mktemp("sa")
    (d / "stub.c").write_text(STUB)
    so = d / "libsa_test.so"
    inc = [f"-I{ROOT / 'include'}", "-I/usr/local/cuda/include", "-I/usr/include"]
    subprocess.run(["gcc", "-O1", "-fPIC", "-shared", "-Wl,-Bsymbolic", *inc, str(ROOT / "csrc/interpose/ccb_nccl_standalone.c"),
                    str(d / "stub.c"), "-o", str(so)], check=True)
    L = ctypes.CDLL(str(so))
    uid = (ctypes.c_char * 128)()
    assert L.ncclGetUniqueId(uid) == 0 and bytes(uid[:4]) == b"ccbs"
    comm = ctypes.c_void_p()

    class Uid(ctypes.Structure):
        _fields_ = [("internal", ctypes.c_char * 128)]

    u = Uid()
    ctypes.memmove(ctypes.byref(u), uid, 128)
    L.ncclCommInitRank.argtypes = [ctypes.POINTER(ctypes.c_void_p), ctypes.c_int, Uid, ctypes.c_int]
    assert L.ncclCommInitRank(ctypes.byref(comm), 4, u, 1) == 0          # rank 1 of 4
    for f in (L.ncclSend, L.ncclRecv):
        f.argtypes = [ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p]
    L.ncclAllReduce.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p]
    L.ncclBroadcast.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p]
    L.ncclAllGather.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p]
    L.stub_get.argtypes = [ctypes.c_int] + [ctypes.POINTER(ctypes.c_int)] * 3 + [ctypes.POINTER(ctypes.c_ulonglong)]

    def log():
        out = []
        for i in range(L.stub_count()):
            k, a, b, n = ctypes.c_int(), ctypes.c_int(), ctypes.c_int(), ctypes.c_ulonglong()
            L.stub_get(i, ctypes.byref(k), ctypes.byref(a), ctypes.byref(b), ctypes.byref(n))
            out.append((k.value, a.value, b.value, n.value))
        L.stub_reset()
        return out

    return L, comm, log


NCCL_INT8, NCCL_INT32, NCCL_FLOAT32, NCCL_FLOAT64 = 0, 2, 7, 8


def test_grouped_sends_and_receives_become_one_call_and_self_pairs_a_copy(provider):
    L, comm, log = provider
    a, b = 0x1000, 0x2000
    assert L.ncclGroupStart() == 0
    assert L.ncclSend(a, 100, NCCL_FLOAT32, 2, comm, None) == 0
    assert L.ncclRecv(b, 100, NCCL_FLOAT32, 0, comm, None) == 0
    assert L.ncclSend(a + 64, 10, NCCL_INT8, 1, comm, None) == 0         # to oneself (this is rank 1)
    assert L.ncclRecv(b + 64, 10, NCCL_INT8, 1, comm, None) == 0
    assert log() == []                                                    # nothing before the group ends
    assert L.ncclGroupEnd() == 0
    assert log() == [(2, 0, 0, 10), (1, 2, 0, 400), (1, 0, 1, 400)]       # the copy, then ONE p2p call with both operations
    assert L.ncclSend(a, 8, NCCL_FLOAT64, 3, comm, None) == 0             # outside a group: at once
    assert log() == [(1, 3, 0, 64)]
    assert L.ncclGroupEnd() != 0                                          # unbalanced
    assert L.ncclGroupStart() == 0 and L.ncclSend(a, 1, NCCL_INT8, 1, comm, None) == 0
    assert L.ncclGroupEnd() != 0 and log() == []                          # a send to oneself without its receive


def test_collectives_choose_the_fused_kernels_the_byte_exchange_or_gather_and_fold(provider):
    L, comm, log = provider
    s, r = 0x10000, 0x20000
    assert L.ncclAllReduce(s, r, 4096, NCCL_FLOAT32, 0, comm, None) == 0
    assert log() == [(3, 0, 0, 4096)]                                     # fp32, sum, no codec: one fused call
    # larger than the stand-in's capacity: cut in halves until the pieces fit, every element once
    assert L.ncclAllReduce(s, r, 3 << 20, NCCL_FLOAT32, 0, comm, None) == 0
    calls = [c for c in log() if c[0] == 3]
    assert sum(c[3] for c in calls if c[3] <= (1 << 20)) == 3 << 20
    # int32 sum: every rank's buffer gathered over the mailbox kernel, then folded
    assert L.ncclAllReduce(s, r, 1000, NCCL_INT32, 0, comm, None) == 0
    got = log()
    assert sorted(g for g in got if g[0] == 1) == sorted([(1, p, d, 4000) for p in (0, 2, 3) for d in (0, 1)])
    assert (2, 0, 0, 4000) in got and got[-1] == (4, 18, 4, 1000)         # own part copied; fold of 4 parts of int32
    # movement of an odd number of bytes: byte exchange, root sends to the three others
    assert L.ncclBroadcast(s, r, 1001, NCCL_INT8, 1, comm, None) == 0     # this rank is the root
    assert sorted(log()) == sorted([(1, p, 0, 1001) for p in (0, 2, 3)] + [(2, 0, 0, 1001)])
    assert L.ncclBroadcast(s, r, 1001, NCCL_INT8, 3, comm, None) == 0     # another root: one receive
    assert log() == [(1, 3, 1, 1001)]
    # movement of whole words goes to the fused exchange as fp32
    assert L.ncclAllGather(s, r, 256, NCCL_INT32, comm, None) == 0
    assert log() == [(3, 0, 3000, 256)]


def test_entry_points_that_are_not_served_say_so(provider):
    import ctypes

    L, comm, _ = provider
    assert L.ncclCommInitAll(None, 2, None) != 0
    L.ncclGetLastError.restype = ctypes.c_char_p
    assert b"one rank per process" in L.ncclGetLastError(None)
    L.ncclGetErrorString.restype = ctypes.c_char_p
    assert L.ncclGetErrorString(0) == b"no error"
    n = ctypes.c_int()
    assert L.ncclCommCount(comm, ctypes.byref(n)) == 0 and n.value == 4
    assert L.ncclCommUserRank(comm, ctypes.byref(n)) == 0 and n.value == 1
