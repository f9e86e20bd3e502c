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
