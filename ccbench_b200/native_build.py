"""Builds the C side of the framework in-tree: the benchmark core, the benchmark
drivers (bin/<arch>/<test>/<test>), helper libraries and interposers (bin/libs/*.so),
tools (bin/<arch>/findso) and daemons (bin/daemons/daemon_<name>).

Output paths are the ones the reference's build scripts produce
(scripts/intermediate/build_tests.sh:144-146, build_comm_wrapper.sh:125,
compile_all.sh:85-120), so run scripts and configs written for it find the same files.
"""
from __future__ import annotations

import os
import shutil
import subprocess
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
BIN = Path(os.environ["CCB_BIN_DIR"]) if os.environ.get("CCB_BIN_DIR") else ROOT / "bin"   # build outputs (default: in-tree)
CUDA = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda"))
INC = [ROOT / "include" / "ccb" / "compat", ROOT / "include", ROOT / "userconfig" / "deviation_metric_examples",
       CUDA / "include"]
CFLAGS = ["-O2", "-g", "-Wall", "-Wno-unused-function", "-Wno-format-truncation", "-fPIC"]

CORE = ["cli.c", "validate.c", "oracle.c", "bindump.c", "perf.c", "devmap.c"]
NCCL_TESTS = ["allreduce", "allgather", "allgatherv", "alltoall", "bcast", "gather", "overlap", "pingpong", "reduce",
              "reducescatter", "scatter", "scatterv"]


def _newer(target: Path, deps) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(Path(d).exists() and Path(d).stat().st_mtime > t for d in deps)


def _run(cmd, verbose):
    if verbose:
        print(" ".join(map(str, cmd)))
    subprocess.run(list(map(str, cmd)), check=True, cwd=ROOT)


def _headers():
    return list((ROOT / "include").rglob("*.h")) + list((ROOT / "csrc").rglob("*.h"))


def have_mpi() -> bool:
    return shutil.which("mpicc") is not None


def metric_sources():
    return sorted((ROOT / "userconfig" / "deviation_metric_examples").glob("*.c"))


def cc(out: Path, srcs, extra=(), shared=False, libs=(), verbose=False, compiler="gcc"):
    out.parent.mkdir(parents=True, exist_ok=True)
    srcs = [Path(s) for s in srcs]
    if not _newer(out, srcs + _headers()):
        return out
    cmd = [compiler, *CFLAGS, *(f"-I{i}" for i in INC), *extra]
    if shared:
        cmd.append("-shared")
    cmd += [*srcs, "-o", out, *libs]
    _run(cmd, verbose)
    return out


def cuda_libs():
    return [f"-L{CUDA / 'lib64'}", "-lcudart", "-Wl,-rpath," + str(CUDA / "lib64")]


def build_c_targets(verbose: bool = False) -> None:
    core = [ROOT / "csrc" / "core" / f for f in CORE]
    metrics = metric_sources()
    libs = BIN / "libs"
    # core as a shared library (loaded by the CPU tests through ctypes)
    cc(libs / "libccb_core.so", core + metrics, shared=True, libs=["-lm", "-ldl", "-lpthread"], verbose=verbose)
    # helper libraries
    cc(libs / "libnccl_extensions.so", [ROOT / "csrc/wrappers/nccl_extensions.c"], shared=True,
       libs=[*cuda_libs(), "-lnccl"], verbose=verbose)
    # NCCL benchmark drivers
    bridge = ROOT / "csrc/core/nccl_bridge.c"
    for t in NCCL_TESTS:
        src = ROOT / "csrc/bench/nccl" / f"{t}.c"
        cu = ROOT / "csrc/bench/nccl" / f"{t}.cu"
        if src.exists():
            cc(BIN / "nccl" / t / t, [src, bridge, *core, *metrics], extra=[f"-I{ROOT / 'csrc/bench/nccl'}"],
               libs=[str(libs / "libnccl_extensions.so"), *cuda_libs(), "-lnccl", "-lm", "-ldl", "-lpthread",
                     "-Wl,-rpath,$ORIGIN/../../libs"], verbose=verbose)
        elif cu.exists():
            out = BIN / "nccl" / t / t
            if _newer(out, [cu, bridge, *core] + _headers()):
                out.parent.mkdir(parents=True, exist_ok=True)
                objs = []
                for c in [bridge, *core, *metrics]:
                    o = ROOT / "build" / "obj" / (c.stem + ".o")
                    cc(o, [c], extra=["-c"], verbose=verbose)
                    objs.append(o)
                _run(["nvcc", "-O2", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
                      *(f"-I{i}" for i in INC), f"-I{ROOT / 'csrc/bench/nccl'}", cu, *objs,
                      str(libs / "libnccl_extensions.so"), "-lnccl", "-lm", "-ldl", "-lpthread",
                      "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN/../../libs", "-o", out], verbose)
    for extra in (ROOT / "ccbench_b200").glob("native_build_*.py"):
        mod = __import__(f"ccbench_b200.{extra.stem}", fromlist=["build"])
        mod.build(verbose=verbose)


if __name__ == "__main__":
    build_c_targets(verbose=True)
