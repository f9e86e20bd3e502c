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


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs >= 2 GPUs")
def test_all_collectives_over_peer_memory():
    n = min(torch.cuda.device_count(), 8)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
           "--master-addr", "127.0.0.1", "--master-port", "29631", os.path.join(HERE, "multigpu_worker.py")]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=900)
    assert p.returncode == 0 and "MULTIGPU_OK" in p.stdout, p.stdout[-3000:] + p.stderr[-3000:]
