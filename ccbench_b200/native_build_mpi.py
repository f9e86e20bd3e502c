"""MPI side: benchmark drivers bin/mpi/<test>/<test>, the MPI interposer, CPU codec
wrappers, perfmpi and mpi_compress_tools. With mpicc on PATH they are built against
the installed MPI; otherwise against the bundled single-host subset (csrc/minimpi),
whose library is then bin/libs/libccb_minimpi.so."""
from __future__ import annotations

from . import native_build as nb

MPI_TESTS = ["allreduce", "allgather", "allgatherv", "alltoall", "bcast", "gather", "overlap", "pingpong", "reduce",
             "reducescatter", "scatter", "scatterv"]


def build(verbose: bool = False) -> None:
    root, libs = nb.ROOT, nb.BIN / "libs"
    real = nb.have_mpi()
    cc = "mpicc" if real else "gcc"
    # with an installed MPI the compiler wrapper brings the include and link flags, and
    # HAVE_MPI tells user code so (the reference's build_tests.sh:118-121 does the same)
    inc, link = (["-DHAVE_MPI"] if real else []), ["-lm", "-ldl", "-lpthread"]
    if not real:
        mini = nb.cc(libs / "libccb_minimpi.so", [root / "csrc/minimpi/minimpi.c"], shared=True, verbose=verbose)
        inc = [f"-I{root / 'csrc/minimpi'}"]
        link = [str(mini), "-Wl,-rpath,$ORIGIN/../../libs", "-Wl,-rpath,$ORIGIN", *link]
    core = [root / "csrc/core" / f for f in nb.CORE] + [root / "csrc/core/mpi_bridge.c"] + nb.metric_sources()
    for t in MPI_TESTS:
        nb.cc(nb.BIN / "mpi" / t / t, [root / "csrc/bench/mpi" / f"{t}.c", *core],
              extra=[*inc, f"-I{root / 'csrc/bench/mpi'}"], libs=link, verbose=verbose, compiler=cc)
    tools = root / "csrc/wrappers/mpi_compress_tools.c"
    ex = root / "userconfig/wrapper_code_examples"
    shared_link = [l for l in link if not l.startswith("-Wl,-rpath,$ORIGIN/../../libs")]
    nb.cc(libs / "libplain_mpi_compress.so", [ex / "communication/plain_mpi_compress/plain_mpi_compress.c", tools], extra=inc,
          shared=True, libs=shared_link, verbose=verbose, compiler=cc)
    nb.cc(libs / "libmpi_zccl_wrapper.so", [ex / "communication/zccl/mpi_zccl_wrapper.c", tools], extra=inc, shared=True,
          libs=shared_link, verbose=verbose, compiler=cc)
    # ZCCL codec replacements and the ZCCL perf wrapper
    nb.cc(libs / "libsz3_for_zccl.so", [ex / "compression/sz3_for_zccl/sz3_for_zccl.c"], shared=True, libs=["-lm", "-ldl"], verbose=verbose)
    nb.cc(libs / "libzfp_for_zccl.so", [ex / "compression/zfp_for_zccl/zfp_for_zccl.c"], shared=True, libs=["-lm", "-ldl"], verbose=verbose)
    nb.cc(libs / "libperfzccl.so", [ex / "perf/perfzccl/perfzccl.c", root / "csrc/wrappers/perf_helper_mpi.c", root / "csrc/core/perf.c"],
          extra=inc, shared=True, libs=shared_link, verbose=verbose, compiler=cc)
    nb.cc(libs / "libmpi_int8.so", [ex / "compression/int8_block/mpi_int8_wrapper.c"], shared=True, libs=["-lm"], verbose=verbose)
    nb.cc(libs / "libmpi_szcpu.so", [ex / "compression/sz_cpu/mpi_szcpu_wrapper.c"], shared=True, libs=["-lm"], verbose=verbose)
    nb.cc(libs / "libmpi_zfp.so", [ex / "compression/zfp/mpi_zfp_wrapper.c"], shared=True, libs=["-lm", "-ldl"], verbose=verbose)
    nb.cc(libs / "libmpi_sz3.so", [ex / "compression/sz3/mpi_sz3_wrapper.c"], shared=True, libs=["-lm", "-ldl"], verbose=verbose)
    nb.cc(libs / "libperfmpi.so", [ex / "perf/perfmpi/perfmpi.c", root / "csrc/wrappers/perf_helper_mpi.c", root / "csrc/core/perf.c"],
          extra=inc, shared=True, libs=shared_link, verbose=verbose, compiler=cc)
