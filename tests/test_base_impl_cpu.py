"""base_ncclXxx reach the library recorded in base_so_name, past anything preloaded: checked
on the CPU with a stand-in library that records what it was called with."""
import ctypes
import subprocess
from pathlib import Path

import pytest

from ccbench_b200.native_build import BIN, ROOT, build_c_targets

FAKE = r'''
#include <stddef.h>
static int calls; static size_t last_count; static void *last_comm; static int last_peer;
int ncclAllReduce(const void*s, void*r, size_t n, int dt, int op, void*c, void*st) { ++calls; last_count = n; last_comm = c; return 0; }
int ncclBroadcast(const void*s, void*r, size_t n, int dt, int root, void*c, void*st) { ++calls; last_count = n; last_comm = c; return 0; }
int ncclReduce(const void*s, void*r, size_t n, int dt, int op, int root, void*c, void*st) { ++calls; last_count = n; last_comm = c; return 0; }
int ncclAllGather(const void*s, void*r, size_t n, int dt, void*c, void*st) { ++calls; last_count = n; last_comm = c; return 0; }
int ncclReduceScatter(const void*s, void*r, size_t n, int dt, int op, void*c, void*st) { ++calls; last_count = n; last_comm = c; return 0; }
int ncclSend(const void*s, size_t n, int dt, int peer, void*c, void*st) { ++calls; last_count = n; last_peer = peer; last_comm = c; return 0; }
int ncclRecv(void*r, size_t n, int dt, int peer, void*c, void*st) { ++calls; last_count = n; last_peer = peer; last_comm = c; return 0; }
int fake_calls(void) { return calls; } size_t fake_count(void) { return last_count; } void *fake_comm(void) { return last_comm; }
int fake_peer(void) { return last_peer; }
'''


@pytest.fixture(scope="module")
def libs(tmp_path_factory):
    build_c_targets()
    d = tmp_path_factory.mktemp("base")
    (d / "fake.c").write_text(FAKE)
    fake = d / "libfake_nccl.so"
    subprocess.run(["gcc", "-shared", "-fPIC", str(d / "fake.c"), "-o", str(fake)], check=True)
    return d, fake


def test_calls_reach_the_recorded_library(libs):
    d, fake = libs
    state = d / "base_so_name"
    state.write_text(str(fake) + "\n")
    base = ctypes.CDLL(str(BIN / "libs" / "libccb_base_impl.so"))
    f = ctypes.CDLL(str(fake))
    f.fake_count.restype = ctypes.c_size_t
    f.fake_comm.restype = ctypes.c_void_p
    assert base.load_base_impl(str(state).encode()) == 0
    vp, sz, i = ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int
    base.base_ncclAllReduce.argtypes = [vp, vp, sz, i, i, vp, vp]
    base.base_ncclSend.argtypes = [vp, sz, i, i, vp, vp]
    base.base_ncclReduceScatter.argtypes = [vp, vp, sz, i, i, vp, vp]
    base.base_nccl_set_comm.argtypes = [vp]
    assert base.base_ncclAllReduce(None, None, 1234, 7, 0, 0x1000, None) == 0
    assert (f.fake_calls(), f.fake_count(), f.fake_comm()) == (1, 1234, 0x1000)
    assert base.base_ncclSend(None, 77, 7, 3, 0x1000, None) == 0 and f.fake_peer() == 3 and f.fake_count() == 77
    base.base_nccl_set_comm(0x2000)          # a fork's wrapped communicator is replaced by the registered one
    assert base.base_ncclReduceScatter(None, None, 5, 7, 0, 0x1000, None) == 0 and f.fake_comm() == 0x2000


def test_missing_record_is_an_error_not_a_crash(tmp_path):
    code = ("import ctypes,sys; b=ctypes.CDLL(sys.argv[1]); rc=b.load_base_impl(sys.argv[2].encode()); "
            "b.base_ncclAllGather.argtypes=[ctypes.c_void_p]*2+[ctypes.c_size_t,ctypes.c_int]+[ctypes.c_void_p]*2; "
            "print(rc, b.base_ncclAllGather(None,None,1,7,None,None))")
    import sys

    r = subprocess.run([sys.executable, "-c", code, str(BIN / "libs" / "libccb_base_impl.so"), str(tmp_path / "absent")],
                       capture_output=True, text=True, cwd=tmp_path)
    assert r.stdout.split() == ["-1", "2"] and "no library recorded" in r.stderr     # 2 = ncclSystemError
