"""User wrapper templates: the ones shipped here, and the reference's own (when its tree is
mounted), must compile against this repository's headers unchanged."""
import os
import shutil
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
TPL = ROOT / "userconfig" / "your_wrapper_code" / "communication"
CUDA_INC = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda")) / "include"
needs_gcc = pytest.mark.skipif(shutil.which("gcc") is None, reason="no gcc")
needs_nccl_h = pytest.mark.skipif(not Path("/usr/include/nccl.h").exists(), reason="no nccl.h")


def _compile(src: Path, tmp_path, *inc):
    out = tmp_path / (src.stem + ".so")
    cmd = ["gcc", "-shared", "-fPIC", "-Wall", "-Werror=implicit-function-declaration", *[f"-I{i}" for i in inc], str(src),
           "-o", str(out), "-ldl"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    return out


def _exports(so: Path):
    out = subprocess.run(["nm", "-D", "--defined-only", str(so)], capture_output=True, text=True, check=True).stdout
    return {line.split()[-1] for line in out.splitlines() if line.strip()}


@needs_gcc
def test_mpi_template_hooks_and_forwards(tmp_path):
    so = _compile(TPL / "user_wrapper_mpi" / "user_wrapper_mpi.c", tmp_path, ROOT / "csrc" / "minimpi")
    assert {"MPI_Allreduce", "MPI_Bcast", "MPI_Reduce", "MPI_Allgather", "MPI_Alltoall"} <= _exports(so)


@needs_gcc
@needs_nccl_h
def test_nccl_templates_hook_the_five_collectives(tmp_path):
    so = _compile(TPL / "user_wrapper_nccl" / "user_wrapper_nccl.c", tmp_path, CUDA_INC)
    assert {"ncclAllReduce", "ncclReduce", "ncclBcast", "ncclBroadcast", "ncclAllGather", "ncclReduceScatter"} <= _exports(so)
    so = _compile(TPL / "user_wrapper_ccb" / "user_wrapper_ccb.c", tmp_path, CUDA_INC, ROOT / "include")
    assert {"ncclAllReduce", "ncclCommDestroy"} <= _exports(so)


@needs_gcc
@pytest.mark.parametrize("kind", ["mpi", "nccl"])
def test_reference_templates_compile_unchanged(tmp_path, kind):
    ref = None
    for base in (os.environ.get("CCB_REFERENCE_DIR", ""), str(ROOT / "baseline" / "_ref" / "CC-Bench"), str(ROOT.parent / "reference")):
        cand = Path(base) / "userconfig" / "your_wrapper_code" / "communication" / f"user_wrapper_{kind}" / f"user_wrapper_{kind}.c"
        if base and cand.exists():
            ref = cand
            break
    if ref is None:
        pytest.skip("reference tree not available")
    if kind == "nccl" and not Path("/usr/include/nccl.h").exists():
        pytest.skip("no nccl.h")
    _compile(ref, tmp_path, ROOT / "csrc" / "minimpi", CUDA_INC)
