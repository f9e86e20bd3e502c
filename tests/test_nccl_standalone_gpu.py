"""The NCCL drivers with every nccl* call served by libccb alone (libccb_nccl_standalone.so
preloaded, no libnccl in the data path): collectives of float go to the fused kernels,
integer and double reductions are gathered over the point-to-point kernel and folded, and
the send/receive drivers run over the peer-arena mailboxes."""
import re
from pathlib import Path

import pytest
import torch

from ccbench_b200.launch import launch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
LIBS = ROOT / "bin" / "libs"
LIB = "libccb_nccl_standalone.so"


def _ranks():
    return min(torch.cuda.device_count(), 4) if torch.cuda.device_count() >= 2 else 1


def _run(tmp_path, test, args, env=None):
    exe = ROOT / "bin" / "nccl" / test / test
    assert exe.exists() and (LIBS / LIB).exists(), "not built (python -m ccbench_b200.cli build)"
    e = {"CCB_ALLOW_SINGLE_RANK": "1", "CCB_VERBOSE": "1", "CCB_ARENA_MB": "512"}
    e.update(env or {})
    rcs, outs = launch(_ranks(), [str(exe), *args], preload=str(LIBS / LIB), env=e, cwd=str(tmp_path), timeout=240, capture=True)
    assert all(rc == 0 for rc in rcs), "\n".join(o or "" for o in outs)[-3000:]
    assert "[ccb_nccl_standalone]" in outs[0], outs[0][-1500:]
    return outs[0]


def _metric(out, name):
    vals = [float(v) for v in re.findall(rf"^\s*{name}: ([-+0-9.eE]+|nan|inf)", out, flags=re.M)]
    assert vals, f"no {name} in:\n{out[-2000:]}"
    return vals


COLLECTIVES = ["allreduce", "allgather", "allgatherv", "alltoall", "bcast", "reduce", "reducescatter", "gather", "scatter", "scatterv"]


@pytest.mark.parametrize("test", COLLECTIVES)
def test_float_collectives_are_exact_without_a_codec(tmp_path, test):
    if test in ("allgatherv", "scatterv") and _ranks() < 2:
        pytest.skip("this driver wants at least two ranks")
    out = _run(tmp_path, test, ["-L", "4096,1048576", "-i", "2", "-w", "1", "-d", "float", "-p", "rank_linear", "-v", "-t", "1e30",
                                "-e", "rel_l2"])
    assert max(_metric(out, "rel_l2")) < 1e-6


@pytest.mark.parametrize("test,dtype", [(t, d) for t in ("allreduce", "reducescatter", "reduce") for d in ("int", "double")] +
                         [(t, d) for t in ("allgather", "alltoall", "bcast") for d in ("int", "double", "char")])
def test_types_the_fused_kernels_do_not_carry(tmp_path, test, dtype):
    """Odd byte counts included (char): movement falls back to the byte exchange over the
    mailbox kernel, reductions to gather-and-fold."""
    out = _run(tmp_path, test, ["-L", "1001,65536", "-i", "2", "-w", "1", "-d", dtype, "-p", "rank_linear", "-v", "-t", "1e30",
                                "-e", "max_abs_err"])
    assert max(_metric(out, "max_abs_err")) == 0


def test_compressed_all_reduce_by_environment(tmp_path):
    out = _run(tmp_path, "allreduce", ["-L", "1048576", "-i", "2", "-w", "1", "-d", "float", "-p", "rank_linear", "-v", "-t", "1e30",
                                       "-e", "rel_l2"], env={"CCB_CODEC": "int8"})
    assert 0 < max(_metric(out, "rel_l2")) < 0.02 or _ranks() == 1


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="point-to-point needs two GPUs")
@pytest.mark.parametrize("test", ["pingpong", "overlap"])
def test_send_and_receive_drivers(tmp_path, test):
    out = _run(tmp_path, test, ["-L", "1048576,33554432", "-i", "3", "-w", "1", "-d", "float"])
    assert "Test Complete" in out or "===" in out, out[-1500:]
