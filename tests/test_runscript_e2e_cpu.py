"""The generated run script, executed: MPI architecture, two CPU ranks, prebuilt wrappers.
Phase 1 runs the benchmark under the compression and communication wrappers, phase 2 again
with the perf wrapper in front; results, perf CSVs and the exit code are checked."""
import csv
import dataclasses
import os
import subprocess
from pathlib import Path

from ccbench_b200 import runscript
from ccbench_b200.config.model import load_config
from ccbench_b200.native_build import build_c_targets

ROOT = Path(__file__).resolve().parent.parent


def test_generated_script_runs_both_phases(tmp_path):
    build_c_targets()
    cfg = load_config(ROOT / "userconfig" / "config_in_jsonc")
    cfg.arch, cfg.benchmark_type, cfg.test_name = "mpi", "mpi_allreduce", "allreduce"
    cfg.job_choice, cfg.nodes, cfg.tasks_per_node = "local", 1, 2
    cfg.msg_mode, cfg.msg_list = "list", [4096, 262144]
    cfg.phase1_warmup = cfg.phase2_warmup = 1
    cfg.phase1_measure = cfg.phase2_measure = 2
    cfg.validation_enabled, cfg.validation_metrics = True, "rel_l2,max_abs_err"
    cfg.output_csv, cfg.output_csv_path = True, str(tmp_path / "results" / "allreduce.csv")
    cfg.daemons_enabled, cfg.selected_daemons, cfg.poll_interval = True, ["cpu"], 0.2
    cfg.phase1_daemons, cfg.phase2_daemons = ["cpu"], ["cpu"]
    cfg.comp = dataclasses.replace(cfg.comp, mode=1, library_paths=["bin/libs/libmpi_int8.so"])
    cfg.comm = dataclasses.replace(cfg.comm, mode=1, library_paths=["bin/libs/libplain_mpi_compress.so"])
    cfg.perf = dataclasses.replace(cfg.perf, mode=1, library_paths=["bin/libs/libperfmpi.so"])
    cfg.env = {"CCB_MINIMPI_JOB": f"e2e{os.getpid()}"}
    script = runscript.write(cfg, ROOT, out_dir=tmp_path)
    env = dict(os.environ, PERF_OUTPUT_DIR=str(tmp_path / "perf_files"), PERF_GENDATA_OUTPUT_DIR=str(tmp_path / "gendata"))
    env.pop("LD_PRELOAD", None)
    r = subprocess.run(["bash", str(script)], capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-2000:]
    out = r.stdout
    assert "Phase 2" in out and "rel_l2" in out
    assert out.index("libmpi_int8.so") < out.index("libplain_mpi_compress.so")
    rows = list(csv.reader(open(cfg.output_csv_path)))
    assert rows[0][0] == "msg_size" and {r[0] for r in rows[1:]} == {"4096", "262144"}
    perf = sorted((tmp_path / "perf_files").glob("perf_function_*.csv"))
    assert len(perf) == 2
    names = {line.split(",")[0] for line in perf[0].read_text().splitlines()[1:]}
    assert {"MPI_Allreduce", "mpi_compress"} <= names
    # the monitoring daemon was started and stopped around the phases and left its samples
    cpu = sorted((tmp_path / "perf_files").glob("perf_cpu*.csv"))
    assert cpu and cpu[0].read_text().startswith("timestamp_sec,")
    assert subprocess.run(["pgrep", "-x", "daemon_cpu"], capture_output=True).returncode != 0, "daemon left running"


def test_capture_run_dumps_buffers_that_feed_a_later_run(tmp_path):
    """benchmark_type = app_gendata: the application (here the MPI all-reduce driver started by
    the local launcher) runs under the perf wrapper, which dumps the buffers of the named call
    and ends the run; the dump directory then serves as a folder data source."""
    build_c_targets()
    cfg = load_config(ROOT / "userconfig" / "config_in_jsonc")
    exe = ROOT / "bin" / "mpi" / "allreduce" / "allreduce"
    cfg.arch, cfg.benchmark_type, cfg.test_name = "mpi", "app_gendata", "allreduce"
    cfg.job_choice, cfg.nodes, cfg.tasks_per_node = "local", 1, 2
    cfg.app_command = f"python3 -m ccbench_b200.launch -n 2 -- {exe} -L 65536 -i 4 -w 1 -d float"
    cfg.gendata_targets = "MPI_Allreduce:2"
    cfg.output_bin_path = str(tmp_path / "captured")
    cfg.daemons_enabled = False
    cfg.comp = dataclasses.replace(cfg.comp, mode=0)
    cfg.comm = dataclasses.replace(cfg.comm, mode=0)
    cfg.perf = dataclasses.replace(cfg.perf, mode=1, library_paths=["bin/libs/libperfmpi.so"])
    cfg.env = {"CCB_MINIMPI_JOB": f"cap{os.getpid()}"}
    script = runscript.write(cfg, ROOT, out_dir=tmp_path)
    env = dict(os.environ, PERF_OUTPUT_DIR=str(tmp_path / "perf_files"), PERF_GENDATA_DONE_DIR=str(tmp_path / "done"))
    env.pop("LD_PRELOAD", None)
    env.pop("PERF_GENDATA_OUTPUT_DIR", None)
    r = subprocess.run(["bash", str(script)], capture_output=True, text=True, timeout=600, env=env)
    dumps = sorted((tmp_path / "captured").rglob("rank_*.bin"))
    assert dumps, r.stdout[-3000:] + r.stderr[-2000:]
    assert {p.name for p in dumps} == {"rank_0.bin", "rank_1.bin"} and dumps[0].parent.name == "MPI_Allreduce_000002"
    assert dumps[0].stat().st_size == 65536
    # the dump directory as the data source of a plain run
    from ccbench_b200 import launch

    rcs, outs = launch.launch(2, [str(exe), "-L", "65536", "-i", "1", "-w", "0", "-d", "float", "-v", "-f", str(dumps[0].parent)], "",
                              {"CCB_MINIMPI_JOB": f"use{os.getpid()}", "DS_TYPE": "folder", "DS_SUFFIX": ".bin", "DS_FORMAT": "binary"},
                              cwd=str(tmp_path), timeout=120, capture=True)
    assert rcs == [0, 0] and "Correct: YES" in outs[0], outs[0][-1500:]
