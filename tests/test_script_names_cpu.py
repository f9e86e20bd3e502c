"""Entry points with the reference's script names exist and start (they forward to the
Python package; reference: scripts/*.sh, scripts/intermediate/*, scripts/statistic/*)."""
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent

SHELL = ["build_script.sh", "compile_all.sh", "configure_modules.sh", "manage_snapshots.sh", "register_daemons.sh",
         "register_job_device_mapper.sh", "register_metrics.sh", "intermediate/build_tests.sh", "intermediate/build_checker.sh",
         "intermediate/build_comm_wrapper.sh", "intermediate/build_comp_wrapper.sh", "intermediate/build_perf_wrapper.sh"]
PYTHON = ["intermediate/generate_iter_datasets.py", "intermediate/generate_4gb_datasets.py", "intermediate/test_dietgpu_compress.py",
          "intermediate/test_dietgpu_all.py", "statistic/draw_hardware.py", "statistic/draw_perf_function.py",
          "statistic/function_analyzer.py"]


@pytest.mark.parametrize("name", SHELL)
def test_shell_entry_points_exist_and_parse(name):
    p = ROOT / "scripts" / name
    assert p.exists() and p.stat().st_mode & 0o111, name
    assert subprocess.run(["bash", "-n", str(p)], capture_output=True).returncode == 0


@pytest.mark.parametrize("name", PYTHON)
def test_python_entry_points_print_their_help(name):
    r = subprocess.run([sys.executable, str(ROOT / "scripts" / name), "--help"], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0 and "usage" in r.stdout.lower(), r.stderr[-500:]


def test_ratio_script_runs_on_the_numpy_codec():
    r = subprocess.run([sys.executable, str(ROOT / "scripts/intermediate/test_dietgpu_all.py"), "--cpu", "--sizes", "8K,64K",
                        "--synthetic-bytes", "64K"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "ratio below 1.0" in r.stdout, r.stderr[-500:]
