"""Real multi-GPU run of every collective (one process per GPU, peer memory over
NVLink). Skipped on boxes with a single GPU, where tests/test_collectives_gpu.py
plays all ranks on one device instead."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def _run(n, sections, port):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(HERE, "multigpu_worker.py")]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=900, env={**os.environ, "CCB_TEST_SECTIONS": sections})
    assert p.returncode == 0 and "MULTIGPU_OK" in p.stdout, p.stdout[-3000:] + p.stderr[-3000:]


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs >= 2 GPUs")
def test_all_collectives_over_peer_memory():
    """Every section of the worker (collectives, pipelined kernel, symmetric memory, point to
    point, overlapping calls, error-bounded codec, MoE) on up to four GPUs."""
    _run(min(torch.cuda.device_count(), 4), "all", 29631)


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() <= 4, reason="needs more than 4 GPUs")
def test_core_collectives_on_every_gpu():
    """The collectives themselves on all GPUs of the box (up to eight)."""
    _run(min(torch.cuda.device_count(), 8), "core", 29632)
