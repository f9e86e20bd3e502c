"""Host description as JSON: hostname, CPUs, memory, GPUs, MPI / NCCL / CUDA
toolchain, InfiniBand, SLURM (what the reference's
.claude/skills/configure-bench/scripts/detect_env.sh:69-410 prints). Read-only."""
from __future__ import annotations

import glob
import os
import platform
import shutil
import subprocess


def _run(cmd, timeout=10) -> str:
    try:
        return subprocess.run(cmd, capture_output=True, text=True, timeout=timeout).stdout.strip()
    except Exception:
        return ""


def detect() -> dict:
    info = {"hostname": platform.node(), "kernel": platform.release(), "cpus": os.cpu_count()}
    try:
        with open("/proc/meminfo") as f:
            info["mem_total_kb"] = int(f.readline().split()[1])
    except Exception:
        pass
    gpus = []
    if shutil.which("nvidia-smi"):
        out = _run(["nvidia-smi", "--query-gpu=index,name,memory.total,driver_version", "--format=csv,noheader"])
        for line in out.splitlines():
            p = [x.strip() for x in line.split(",")]
            if len(p) >= 4:
                gpus.append({"index": int(p[0]), "name": p[1], "memory": p[2], "driver": p[3]})
    info["gpus"] = gpus
    info["nvcc"] = _run(["nvcc", "--version"]).splitlines()[-1] if shutil.which("nvcc") else None
    info["mpi"] = {"mpicc": shutil.which("mpicc"), "mpirun": shutil.which("mpirun")}
    nccl = sorted(glob.glob("/usr/lib/x86_64-linux-gnu/libnccl.so*") + glob.glob("/usr/local/lib/libnccl.so*"))
    info["nccl"] = {"libraries": nccl, "header": os.path.exists("/usr/include/nccl.h")}
    info["infiniband"] = sorted(os.listdir("/sys/class/infiniband")) if os.path.isdir("/sys/class/infiniband") else []
    info["slurm"] = {"srun": shutil.which("srun"), "sbatch": shutil.which("sbatch"), "job_id": os.environ.get("SLURM_JOB_ID")}
    plug = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "plugin_projects")
    info["plugins"] = sorted(os.listdir(plug)) if os.path.isdir(plug) else []
    return info
