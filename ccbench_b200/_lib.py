"""Loader and builder of the native libraries (in-tree, never JIT-cached).

`libccb.so` holds the host runtime and every fused sm_100a kernel; it is built by
`build_native()` with plain nvcc and loaded with ctypes, so no torch extension and
no JIT cache is involved and the built file travels with the source tree.
"""
from __future__ import annotations

import ctypes
import os
import shutil
import subprocess
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
NATIVE_DIR = Path(__file__).resolve().parent / "_native"
LIBCCB = NATIVE_DIR / "libccb.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-shared", "--threads", "0",
]

RT_SOURCES = ["csrc/rt/ccb_rt.cu", "csrc/rt/ccb_bootstrap.cpp", "csrc/kernels/ccb_standalone.cu",
              "csrc/kernels/ccb_sz.cu", "csrc/kernels/ccb_moe.cu", "csrc/kernels/ccb_noalloc.cu", "csrc/kernels/ccb_pipe.cu",
              "csrc/kernels/ccb_lossless.cu"]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; libccb.so cannot be built")
    return exe


def _stale(target: Path, sources: list[Path]) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(s.exists() and s.stat().st_mtime > t for s in sources)


def build_native(force: bool = False, verbose: bool = False) -> Path:
    """Compile libccb.so for sm_100a if it is missing or older than its sources."""
    NATIVE_DIR.mkdir(parents=True, exist_ok=True)
    srcs = [ROOT / s for s in RT_SOURCES if (ROOT / s).exists()]
    deps = srcs + list((ROOT / "csrc").rglob("*.cuh")) + list((ROOT / "csrc").rglob("*.h")) + list((ROOT / "include").rglob("*.h"))
    if force or _stale(LIBCCB, deps):
        cmd = [_nvcc(), *NVCC_FLAGS, f"-I{ROOT / 'include'}", *map(str, srcs), "-o", str(LIBCCB)]
        if verbose:
            print(" ".join(cmd))
        subprocess.run(cmd, check=True, cwd=ROOT)
    return LIBCCB


_lib = None


def lib() -> ctypes.CDLL:
    """The loaded libccb.so (built on first use when missing)."""
    global _lib
    if _lib is None:
        if not LIBCCB.exists():
            build_native()
        _lib = ctypes.CDLL(str(LIBCCB))
        _declare(_lib)
    return _lib


def _declare(L: ctypes.CDLL) -> None:
    c_u64, c_int, c_vp = ctypes.c_uint64, ctypes.c_int, ctypes.c_void_p
    pp = ctypes.POINTER(ctypes.c_void_p)
    L.ccb_last_error.restype = ctypes.c_char_p
    L.ccb_launch_count.restype = c_u64
    L.ccb_comm_create.argtypes = [pp, c_int, c_int, ctypes.c_char_p, c_u64, c_int]
    L.ccb_comm_create_local.argtypes = [pp, c_int, c_u64]
    L.ccb_comm_destroy.argtypes = [c_vp]
    for f in ("ccb_comm_rank", "ccb_comm_nranks", "ccb_comm_nlocal", "ccb_comm_has_nvls"):
        getattr(L, f).argtypes = [c_vp]
    L.ccb_comm_arena_bytes.argtypes = [c_vp]
    L.ccb_comm_arena_bytes.restype = c_u64
    L.ccb_comm_set_timeout_ms.argtypes = [c_vp, c_u64]
    L.ccb_comm_set_max_ctas.argtypes = [c_vp, c_int]
    L.ccb_comm_status.argtypes = [c_vp, ctypes.POINTER(ctypes.c_uint32)]
    L.ccb_wire_bytes.argtypes = [c_int, c_int, c_u64]
    L.ccb_wire_bytes.restype = c_u64
    L.ccb_p2p.argtypes = [c_vp, c_vp, c_int, c_vp]
    L.ccb_link_probe.argtypes = [c_vp, c_int, c_int, c_u64, c_vp]
    L.ccb_fold.argtypes = [c_int, c_int, c_vp, c_u64, c_int, c_u64, c_vp, c_vp]
    L.ccb_all_reduce.argtypes = [c_vp, pp, pp, c_u64, c_int, c_int, c_int, c_int, pp, c_vp]
    L.ccb_reduce_scatter.argtypes = [c_vp, pp, pp, c_u64, c_int, c_int, c_int, pp, c_vp]
    L.ccb_reduce.argtypes = [c_vp, pp, pp, c_u64, c_int, c_int, c_int, c_int, c_vp]
    up = ctypes.POINTER(c_u64)
    L.ccb_exchange.argtypes = [c_vp, pp, pp, up, up, up, c_int, c_int, c_vp]
    L.ccb_all_gather.argtypes = [c_vp, pp, pp, c_u64, c_int, c_int, c_vp]
    L.ccb_broadcast.argtypes = [c_vp, pp, pp, c_u64, c_int, c_int, c_int, c_vp]
    L.ccb_all_to_all.argtypes = [c_vp, pp, pp, c_u64, c_int, c_int, c_vp]
    L.ccb_scatter.argtypes = [c_vp, pp, pp, c_u64, c_int, c_int, c_int, c_vp]
    L.ccb_gather.argtypes = [c_vp, pp, pp, c_u64, c_int, c_int, c_int, c_vp]
