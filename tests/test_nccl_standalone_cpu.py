"""The NCCL-free provider exports every nccl* symbol that the benchmark drivers and the
extension library import, so preloading it leaves no call for libnccl."""
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
LIB = ROOT / "bin" / "libs" / "libccb_nccl_standalone.so"


def _symbols(path, defined):
    flag = "--defined-only" if defined else "--undefined-only"
    out = subprocess.run(["nm", "-D", flag, str(path)], capture_output=True, text=True, check=True).stdout
    return {line.split()[-1].split("@")[0] for line in out.splitlines() if line.strip()}


def test_every_nccl_symbol_the_drivers_import_is_served():
    drivers = sorted((ROOT / "bin" / "nccl").glob("*/*"))
    if not LIB.exists() or not drivers:
        pytest.skip("native side not built (python -m ccbench_b200.cli build)")
    have = _symbols(LIB, True)
    assert not any(s.startswith("nccl") for s in _symbols(LIB, False)), "the provider itself must not import NCCL"
    ext = ROOT / "bin" / "libs" / "libnccl_extensions.so"
    served_by_extensions = _symbols(ext, True) if ext.exists() else set()
    missing = {}
    for exe in [*drivers, *([ext] if ext.exists() else [])]:
        if exe.is_file():
            want = {s for s in _symbols(exe, False) if s.startswith("nccl")}
            lack = want - have - served_by_extensions
            if lack:
                missing[exe.name] = sorted(lack)
    assert not missing, missing
