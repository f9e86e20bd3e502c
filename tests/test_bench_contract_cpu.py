"""The parts of the bench.py contract that can be checked without a GPU."""
import json
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def test_reference_arm_at_one_rank_reports_unavailable():
    r = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "1"],
                       capture_output=True, text=True, timeout=300, cwd=ROOT)
    assert r.returncode == 0, r.stderr[-2000:]
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and "unavailable" in line and "\n" not in line["unavailable"]


def test_flags_and_defaults():
    out = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--help"], capture_output=True, text=True, timeout=120).stdout
    for flag in ("--gpus", "--steps", "--warmup", "--impl", "--via", "--no-call-overlap"):
        assert flag in out
    src = (ROOT / "bench.py").read_text()
    for key in ('"metric"', '"value"', '"unit"', '"n_gpus"', '"steps"', '"warmup"', '"ms_per_step"', '"higher_is_better"', '"scaling"',
                '"vs_baseline"', '"dtype"', '"data"', '"config"', '"clocks"', '"e2e"', '"gpu_launches"', '"h2d_bytes_per_step"',
                '"d2h_bytes_per_step"', '"serialised_ms_per_step"', '"pipelined_kernel"', '"call_overlap"', '"metric_readback"', '"copy_schedule"',
                '"fraction_of_sm_store_rate_695"'):
        assert key in src, key


def test_graft_entry_points_exist():
    sys.path.insert(0, str(ROOT))
    import __graft_entry__ as g

    assert callable(g.build) and callable(g.smoke)
