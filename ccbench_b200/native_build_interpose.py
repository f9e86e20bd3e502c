"""Builds the interposers and wrapper helper libraries into bin/libs."""
from __future__ import annotations

from . import native_build as nb
from ._lib import LIBCCB, build_native


def build(verbose: bool = False) -> None:
    root, libs = nb.ROOT, nb.BIN / "libs"
    build_native(verbose=verbose)
    # libccb.so is copied next to the interposer so that $ORIGIN finds it
    dst = libs / "libccb.so"
    if nb._newer(dst, [LIBCCB]):
        libs.mkdir(parents=True, exist_ok=True)
        dst.write_bytes(LIBCCB.read_bytes())
        dst.chmod(0o755)
    rpath = ["-Wl,-rpath,$ORIGIN"]
    nb.cc(libs / "libccb_nccl.so", [root / "csrc/interpose/ccb_nccl_interpose.c"], shared=True,
          libs=[str(dst), *nb.cuda_libs(), "-ldl", "-lpthread", *rpath], verbose=verbose)
    # NCCL's API on libccb alone (no libnccl underneath): the role of the reference's NCCL-replacement wrapper
    nb.cc(libs / "libccb_nccl_standalone.so", [root / "csrc/interpose/ccb_nccl_standalone.c"], shared=True,
          libs=[str(dst), *nb.cuda_libs(), "-lpthread", *rpath], verbose=verbose)
    for name, src, extra in [
        ("libnccl_compress_tools.so", root / "csrc/wrappers/nccl_compress_tools.c", [*nb.cuda_libs(), "-lnccl"]),
        ("libccb_coccl_hooks.so", root / "csrc/wrappers/coccl_hooks.c", [str(dst), *nb.cuda_libs(), *rpath]),
        # lossless float codec behind the same four hooks (the reference's DietGPU wrapper role)
        ("libdietgpu_wrapper.so", root / "userconfig/wrapper_code_examples/compression/dietgpu/dietgpu.c",
         [str(dst), *nb.cuda_libs(), *rpath]),
        # error-bounded GPU codec behind the four hooks (the reference's cuZFP wrapper role)
        ("libzfp_for_gpu_nvidia.so", root / "userconfig/wrapper_code_examples/compression/zfp_for_gpu_nvidia/zfp_for_gpu_nvidia.c",
         [str(dst), *nb.cuda_libs(), "-lm", *rpath]),
    ]:
        if src.exists():
            nb.cc(libs / name, [src], shared=True, libs=extra, verbose=verbose)
    # loader of the library under the preload chain (base_ncclXxx)
    base = root / "csrc/core/base_impl.c"
    if base.exists():
        nb.cc(libs / "libccb_base_impl.so", [base], shared=True, libs=["-ldl"], verbose=verbose)
    # perf wrapper for the NCCL path: plain cc, no CUDA or NCCL headers
    perf_src = [root / "userconfig/wrapper_code_examples/perf/perfnccl/perfnccl.c",
                root / "csrc/wrappers/perf_helper_nccl.c", root / "csrc/core/perf.c"]
    if all(p.exists() for p in perf_src):
        nb.cc(libs / "libperfnccl.so", perf_src, shared=True, libs=["-ldl", "-lpthread"], verbose=verbose, compiler="cc")
    # example compression wrapper with its own kernels (4-bit / 8-bit groups, SDP4Bit chunk layout)
    import shutil

    nvcc = shutil.which("nvcc") or str(nb.CUDA / "bin" / "nvcc")
    for src, name in [
        (root / "userconfig/wrapper_code_examples/compression/sdp4bit/sdp4bit.cu", "libsdp4bit.so"),
        # the user template of the four hooks, built with its example codec so that it is tested
        (root / "userconfig/wrapper_code_examples/compression/coccl_wrapper_template.cu", "libcoccl_wrapper_template.so"),
    ]:
        out = libs / name
        if src.exists() and nb._newer(out, [src]):
            nb._run([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-shared", "-Xcompiler", "-fPIC",
                     *(f"-I{i}" for i in nb.INC), src, "-o", out], verbose)
