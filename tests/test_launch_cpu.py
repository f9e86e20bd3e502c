"""The local launcher: rank environment, preload, output capture, time limit."""
import sys

from ccbench_b200.launch import launch


def test_ranks_get_their_environment_and_directories(tmp_path):
    code = ("import os; print(os.environ['OMPI_COMM_WORLD_RANK'], os.environ['OMPI_COMM_WORLD_SIZE'], "
            "os.environ['OMPI_COMM_WORLD_LOCAL_RANK'], os.environ.get('EXTRA'), os.environ.get('LD_PRELOAD', ''))")
    rcs, outs = launch(3, [sys.executable, "-c", code], preload="", env={"EXTRA": "x"}, cwd=str(tmp_path), timeout=60, capture=True)
    assert rcs == [0, 0, 0]
    assert [o.split()[:4] for o in outs] == [[str(r), "3", str(r), "x"] for r in range(3)]
    assert (tmp_path / "nccl_id_file").is_dir() and (tmp_path / "runtime_files" / "nccl_agg").is_dir()


def test_stale_rendezvous_files_are_removed(tmp_path):
    d = tmp_path / "nccl_id_file"
    d.mkdir()
    (d / "nccl_bench_id").write_bytes(b"old")
    launch(1, [sys.executable, "-c", "pass"], cwd=str(tmp_path), timeout=60, capture=True)
    assert not (d / "nccl_bench_id").exists()


def test_a_rank_that_hangs_is_ended_by_the_time_limit(tmp_path):
    code = "import os, time; time.sleep(60 if os.environ['OMPI_COMM_WORLD_RANK'] == '1' else 0)"
    rcs, _ = launch(2, [sys.executable, "-c", code], cwd=str(tmp_path), timeout=3, capture=True)
    assert rcs[0] == 0 and rcs[1] != 0
