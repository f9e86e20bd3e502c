"""Failure detection on the host, with no GPU involved: what the ranks of a communicator
see during the rendezvous when a peer never joins or leaves half-way. Ranks are child
processes; the failures are made by not starting a rank or by having it return early."""
import ctypes
import multiprocessing as mp
import os
import time
import uuid

import pytest

from ccbench_b200._lib import lib


def _rank(rank, nranks, tag, timeout_ms, skip_barrier, q, gate):
    L = lib()
    L.ccb_test_bootstrap_exchange.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_char_p, ctypes.c_int, ctypes.c_int,
                                              ctypes.POINTER(ctypes.c_int), ctypes.c_char_p, ctypes.c_int]
    s = ctypes.c_int(-1)
    err = ctypes.create_string_buffer(256)
    gate.wait(timeout=120)   # children start the rendezvous together, however long their imports took
    t0 = time.time()
    rc = L.ccb_test_bootstrap_exchange(rank, nranks, tag.encode(), timeout_ms, skip_barrier, ctypes.byref(s), err, 256)
    q.put((rank, rc, s.value, err.value.decode(), time.time() - t0))


def _run(nranks, started, timeout_ms=1500, leaves_early=()):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    tag = "t" + uuid.uuid4().hex[:10]
    started = list(started)
    gate = ctx.Barrier(len(started))
    procs = [ctx.Process(target=_rank, args=(r, nranks, tag, timeout_ms, 1 if r in leaves_early else 0, q, gate)) for r in started]
    for p in procs:
        p.start()
    out = {}
    for _ in procs:
        r, rc, s, err, dt = q.get(timeout=180)
        out[r] = (rc, s, err, dt)
    for p in procs:
        p.join(timeout=30)
    return out


def test_all_ranks_join_and_descriptors_travel():
    out = _run(4, range(4), timeout_ms=20000)
    assert all(rc == 0 and s == 0 + 1 + 2 + 3 for rc, s, _, _ in out.values()), out


def test_a_rank_that_never_joins_ends_the_rendezvous_with_an_error():
    out = _run(3, [0, 1], timeout_ms=1200)
    for rc, _, err, dt in out.values():
        assert rc == 1 and err, out
        assert dt < 10, "the wait must be bounded by the time limit"


def test_a_rank_that_leaves_before_the_barrier_is_noticed_by_the_others():
    out = _run(3, range(3), timeout_ms=2500, leaves_early=(2,))
    assert out[2][0] == 0
    for r in (0, 1):
        rc, s, err, dt = out[r]
        assert rc == 1 and "barrier" in err and s == 3 and dt < 10, out
