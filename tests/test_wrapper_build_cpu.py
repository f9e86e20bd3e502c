"""The wrapper builder: modes 0-3 of the three selection files, as the reference's
build_{comm,comp,perf}_wrapper.sh define them."""
import subprocess
from pathlib import Path

import pytest

from ccbench_b200.config.model import WrapperSel, load_config
from ccbench_b200.wrapper_build import build_wrapper

ROOT = Path(__file__).resolve().parent.parent
TPL = "userconfig/your_wrapper_code/communication"


def _sel(mode, name, **kw):
    base = dict(mode=mode, library_paths=[], source_files=[], source_dirs=[], include_files=[], include_dirs=[], libraries=[],
                output_name=name)
    base.update(kw)
    return WrapperSel(**base)


def _exports(so):
    out = subprocess.run(["nm", "-D", "--defined-only", str(so)], capture_output=True, text=True, check=True).stdout
    return {line.split()[-1] for line in out.splitlines() if line.strip()}


@pytest.fixture
def cleanup():
    made = []
    yield made
    for p in made:
        Path(p).unlink(missing_ok=True)


def test_modes_0_and_1_build_nothing():
    assert build_wrapper("comm", _sel(0, "x.so"), "nccl") is None
    assert build_wrapper("comm", _sel(1, "x.so", library_paths=["bin/libs/libccb_nccl.so"]), "nccl") is None


def test_default_perf_selection_builds_from_the_reference_paths(cleanup):
    cfg = load_config(ROOT / "userconfig" / "config_in_jsonc")
    assert cfg.perf.mode == 3 and any(s.startswith("run_codes/") for s in cfg.perf.source_files)
    sel = _sel(3, "libtest_perf_build.so", source_files=cfg.perf.source_files, source_dirs=cfg.perf.source_dirs,
               include_files=cfg.perf.include_files)
    out = build_wrapper("perf", sel, "nccl")
    cleanup.append(out)
    assert {"ncclAllReduce", "ncclSend", "ncclCompress"} <= _exports(out)


def test_user_templates_build_from_source(cleanup):
    out = build_wrapper("comm", _sel(3, "libtest_user_nccl.so", source_files=[f"{TPL}/user_wrapper_nccl/user_wrapper_nccl.c"]), "nccl")
    cleanup.append(out)
    assert "ncclAllReduce" in _exports(out)
    out = build_wrapper("comm", _sel(3, "libtest_user_mpi.so", source_files=[f"{TPL}/user_wrapper_mpi/user_wrapper_mpi.c"]), "mpi")
    cleanup.append(out)
    assert "MPI_Allreduce" in _exports(out)


def test_mode_2_links_the_listed_libraries(cleanup):
    sel = _sel(2, "libtest_mode2.so", source_files=[f"{TPL}/user_wrapper_ccb/user_wrapper_ccb.c"],
               library_paths=["ccbench_b200/_native/libccb.so"])
    out = build_wrapper("comm", sel, "nccl")
    cleanup.append(out)
    needed = subprocess.run(["readelf", "-d", str(out)], capture_output=True, text=True).stdout
    assert "libccb.so" in needed and "ncclAllReduce" in _exports(out)


def test_missing_sources_and_names_are_reported(capsys):
    assert build_wrapper("comm", _sel(3, "libnone.so", source_files=["does/not/exist.c"]), "nccl") is None
    assert "no source files" in capsys.readouterr().out
    with pytest.raises(ValueError):
        build_wrapper("comm", _sel(3, "", source_files=[f"{TPL}/user_wrapper_nccl/user_wrapper_nccl.c"]), "nccl")


def test_the_installed_mpi_path_builds_with_a_compiler_wrapper(tmp_path):
    """No MPI is installed here, so a stand-in `mpicc` (a script that adds the include and
    link flags of the bundled MPI subset, which is what a real compiler wrapper does for its
    MPI) is put on PATH: the MPI drivers and wrappers must then be compiled by it, with
    -DHAVE_MPI, into a separate output directory, and the result must run."""
    import os
    import stat
    import subprocess
    import sys

    from ccbench_b200.native_build import ROOT, build_c_targets

    build_c_targets()   # the stand-in links the prebuilt subset library
    mini = ROOT / "bin" / "libs" / "libccb_minimpi.so"
    assert mini.exists()
    stub_dir, log = tmp_path / "stub", tmp_path / "mpicc.log"
    stub_dir.mkdir()
    stub = stub_dir / "mpicc"
    stub.write_text(f"""#!/bin/sh
echo "$@" >> {log}
exec gcc -I{ROOT / 'csrc/minimpi'} "$@" {mini} -Wl,-rpath,{mini.parent}
""")
    stub.chmod(stub.stat().st_mode | stat.S_IEXEC)
    env = dict(os.environ, PATH=f"{stub_dir}:{os.environ['PATH']}", CCB_BIN_DIR=str(tmp_path / "bin"), PYTHONPATH=str(ROOT))
    r = subprocess.run([sys.executable, "-c", "from ccbench_b200 import native_build_mpi as m; m.build()"], env=env, cwd=ROOT,
                       capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    calls = log.read_text().splitlines()
    drivers = [c for c in calls if "csrc/bench/mpi/allreduce.c" in c]
    assert drivers and all("-DHAVE_MPI" in c for c in drivers)
    assert any("plain_mpi_compress.c" in c and "-shared" in c for c in calls)
    assert any("perfmpi.c" in c for c in calls)
    assert not (tmp_path / "bin" / "libs" / "libccb_minimpi.so").exists(), "the bundled subset is not built when an MPI is installed"
    exe = tmp_path / "bin" / "mpi" / "allreduce" / "allreduce"
    assert exe.exists()
    run = subprocess.run([sys.executable, "-m", "ccbench_b200.launch", "-n", "2", "--", str(exe), "-L", "4096", "-i", "1", "-w", "0",
                          "-d", "double", "-v"], env=dict(env, CCB_MINIMPI_JOB=f"stub{os.getpid()}"), cwd=tmp_path,
                         capture_output=True, text=True, timeout=120)
    assert run.returncode == 0 and "Correct: YES" in run.stdout, run.stdout[-1500:] + run.stderr[-1500:]
    # the wrapper builder picks the compiler wrapper for MPI wrappers too
    code = ("import dataclasses\n"
            "from ccbench_b200.config.model import load_config\n"
            "from ccbench_b200.wrapper_build import build_wrapper\n"
            "from ccbench_b200.native_build import ROOT\n"
            "cfg = load_config(ROOT / 'userconfig' / 'config_in_jsonc')\n"
            "sel = dataclasses.replace(cfg.comm, mode=3, output_name='libstub_mpicc_probe.so', source_dirs=[], include_files=[], "
            "include_dirs=[], libraries=[], library_paths=[], source_files=['userconfig/wrapper_code_examples/communication/"
            "plain_mpi_compress/plain_mpi_compress.c', 'csrc/wrappers/mpi_compress_tools.c'])\n"
            "print(build_wrapper('comm', sel, 'mpi'))\n")
    try:
        r = subprocess.run([sys.executable, "-c", code], env=env, cwd=ROOT, capture_output=True, text=True, timeout=300)
        assert r.returncode == 0, r.stderr[-2000:]
        assert any("plain_mpi_compress.c" in c and "libstub_mpicc_probe.so" in c for c in log.read_text().splitlines())
    finally:
        probe = ROOT / "bin" / "libs" / "libstub_mpicc_probe.so"
        if probe.exists():
            probe.unlink()


@pytest.mark.parametrize("folder,symbols", [
    ("plain_nccl_compress", {"ncclAllReduce", "ncclReduceScatter", "ncclSend", "ncclGroupEnd"}),
    ("nccl_via_uccl", {"ncclGetUniqueId", "ncclCommInitRank", "ncclAllReduce", "ncclSend", "ncclRecv", "ncclGroupStart"}),
])
def test_reference_wrapper_folders_build_in_mode_3(cleanup, folder, symbols):
    """A configuration that still names the reference's communication-wrapper folders in
    source_dirs builds the corresponding wrapper of this repository, linked with libccb."""
    if not (ROOT / "bin/libs/libccb.so").exists():
        pytest.skip("native side not built (python -m ccbench_b200.cli build)")
    name = f"libtest_{folder}.so"
    out = build_wrapper("comm", _sel(3, name, source_dirs=[f"userconfig/wrapper_code_examples/communication/{folder}"]), "nccl")
    cleanup.append(out)
    assert out is not None and symbols <= _exports(out)
    needed = subprocess.run(["readelf", "-d", str(out)], capture_output=True, text=True).stdout
    assert "libccb.so" in needed
