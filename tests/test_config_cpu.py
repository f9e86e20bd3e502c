"""JSONC reader, configuration model, run-script generator, snapshots, analysis and
daemons (CPU only)."""
import json
import os
import subprocess
import sys
import time

import pytest

from ccbench_b200 import runscript, snapshots
from ccbench_b200.config import jsonc_loads, load_config

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CFG = os.path.join(ROOT, "userconfig/config_in_jsonc")


def test_jsonc_keeps_comment_markers_inside_strings():
    text = """
    { // line comment
      "url": "http://host//path", /* block
      comment */ "cmd": "a /* not a comment */ b",
      "list": [1, 2, 3, ],   // trailing comma
      "nested": { "k": "v", },
    }"""
    d = jsonc_loads(text)
    assert d["url"] == "http://host//path" and d["cmd"] == "a /* not a comment */ b"
    assert d["list"] == [1, 2, 3] and d["nested"] == {"k": "v"}


def test_reference_style_config_files_load(tmp_path):
    """A configuration directory written for the reference (its keys, its comment style)."""
    (tmp_path / "bench_basic_config.jsonc").write_text("""{
      "benchmark_type": "mpi_allreduce", "communication_arch": "mpi", // arch
      "data_source": {"type": "file", "file_path": "dataset/weight/weight_4gb.f32", "pattern_type": "rank_linear",
                      "offset_config": {"base_offset": 0, "per_rank_offset": false, "custom_offsets": []}},
      "output": {"csv": true, "csv_path": "results/pingpong.csv", "binary": true, "bin_path": "results/AllReduce"},
      "mpi_operation": {"datatype": "MPI_FLOAT"},
      "iterations": {"performance": {"warmup": 3, "measurement": 5}, "perf_round": {"warmup": 1, "measurement": 2}},
      "message_sizes": {"mode": "list", "min": 1, "max": 2, "increment": 2, "increment_type": "add", "list": [8388608, 40894464]},
      "gendata_capture": {"targets": [{"operation": "all", "occurrence": [3, 16]}]}
    }""")
    (tmp_path / "job_config.jsonc").write_text('{"job_choice": "mpirun", "cross_alloc_nodes": ["n1", "n2"], "slurm": {"resources": {"nodes": 2, "tasks_per_node": 8}}}')
    (tmp_path / "perf_kernel_selection.jsonc").write_text('{"mode": 3, "source_dirs": ["userconfig/wrapper_code_examples/perf/perfmpi"], "output_name": "libperfmpi.so"}')
    (tmp_path / "environment_variables.jsonc").write_text('{"UCX_TLS": "rc,self,sm", "ALLGATHERV_WEIGHTS": "1,2,3,4"}')
    (tmp_path / "deviation_config.jsonc").write_text('{"validation": {"enabled": true, "selected_metrics": "mse, mae, cos_sim"}}')
    (tmp_path / "daemon_config.jsonc").write_text('{"selected_daemons": "cpu, gpu_nvidia", "performance": {"enabled": true, "phase1_daemons": "gpu_nvidia", "phase2_daemons": "gpu_nvidia,stress_gpu_nvidia", "poll_interval_sec": 0.5}, "stress": {"cpu_percent": 0, "gpu_percent": 60}}')
    cfg = load_config(tmp_path)
    assert (cfg.arch, cfg.test_name, cfg.nprocs, cfg.datatype) == ("mpi", "allreduce", 16, "float")
    assert cfg.gendata_targets == "all:3,16" and cfg.validation_metrics == "mse,mae,cos_sim"
    assert cfg.phase2_daemons == ["gpu_nvidia", "stress_gpu_nvidia"] and cfg.stress_gpu_percent == 60
    script = runscript.generate(cfg, ROOT)
    assert "mpirun --hostfile $CROSS_HOSTFILE -np 16 --map-by node --bind-to none -x LD_LIBRARY_PATH -x LD_PRELOAD -x UCX_TLS -x ALLGATHERV_WEIGHTS" in script
    assert '-L 8388608,40894464 -i 5 -w 3 -p rank_linear -v -e "mse,mae,cos_sim" -f "dataset/weight/weight_4gb.f32" -d float -c -o "results/pingpong.csv" -b -B "results/AllReduce"' in script
    assert "-i 2 -w 1" in script  # phase 2 uses the perf-round counts
    assert "export DS_PER_RANK_OFFSET=false" in script and "export STRESS_GPU_PERCENT=60" in script
    assert 'echo "n1 slots=8" >> "$CROSS_HOSTFILE"' in script
    assert script.index("libperfmpi.so") > script.index("Phase 2")  # the perf wrapper only joins in phase 2
    assert "daemon_stress_gpu_nvidia" in script.split("Phase 2")[1] and "daemon_stress_gpu_nvidia" not in script.split("Phase 2")[0]
    assert subprocess.run(["bash", "-n"], input=script, text=True).returncode == 0


def test_default_config_generates_every_launcher(tmp_path):
    cfg = load_config(CFG)
    assert cfg.arch == "nccl" and cfg.comm.mode == 1
    for choice, name in runscript.SCRIPT_NAMES.items():
        cfg.job_choice = choice
        p = runscript.write(cfg, ROOT, out_dir=tmp_path)
        assert p.name == name and os.access(p, os.X_OK)
        text = p.read_text()
        assert subprocess.run(["bash", "-n", str(p)]).returncode == 0
        order = [text.index("compression") if "compression:" in text else -1, text.index("libccb_nccl.so"), text.index("libnccl_extensions.so")]
        assert order[1] < order[2]
        if choice == "slurm":
            assert "#SBATCH --nodes=1" in text and "srun --nodes=1 --ntasks=8" in text
        if choice == "local":
            assert "python3 -m ccbench_b200.launch -n 8 --" in text


def test_snapshots_roundtrip(tmp_path, monkeypatch):
    monkeypatch.setattr(snapshots, "ROOT", tmp_path)
    cfgdir = tmp_path / "cfg"
    cfgdir.mkdir()
    for f in os.listdir(CFG):
        (cfgdir / f).write_text(open(os.path.join(CFG, f)).read())
    d = snapshots.save("base", cfgdir, level="summary", description="first")
    meta = json.loads((d / "metadata.json").read_text())
    assert set(meta) == {"snapshot_level", "timestamp", "git_commit", "description"} and meta["description"] == "first"
    assert (d / "DESCRIPTION.md").exists() and (d / "effective_config.json").exists()
    (cfgdir / "deviation_config.jsonc").write_text('{"validation": {"enabled": false, "selected_metrics": "mse"}}')
    diff = snapshots.compare("base", "current", config_dir=cfgdir)
    assert "deviation_config.jsonc" in diff and '"enabled": false' in diff
    snapshots.load("base", cfgdir)
    assert load_config(cfgdir).validation_enabled
    assert [n for n, _ in snapshots.list_snapshots()] == ["base"]
    snapshots.delete("base")
    assert snapshots.list_snapshots() == []


def test_function_analyzer_sweep(tmp_path):
    from ccbench_b200.analysis import function_analyzer as fa

    (tmp_path / "perf_function_0.csv").write_text(
        "func_name,timestamp_us,call_count,duration,msg_bytes,intra\n"
        "MPI_Allreduce,0.000000,1.000000,0.000100,,\n"          # comm   0..100 us
        "mpi_compress,50.000000,1.000000,0.000100,,\n"            # comp  50..150 us (overlap 50..100)
        "MPI_Isend,300.000000,1.000000,0.000002,1048576.000000,1.000000\n")  # async: estimated from pingpong
    (tmp_path / "pingpong.csv").write_text("msg_size,partner,latency_us,bandwidth_gbps,send0_us,recv0_us,recvP_us,sendP_us\n"
                                           "524288,1,10,1,20.00,20.00,20,20\n2097152,1,10,1,80.00,80.00,80,80\n")
    res = fa.analyze(str(tmp_path), str(tmp_path / "pingpong.csv"))["0"]
    assert abs(res["overlap"] - 50) < 1e-6 and abs(res["comp"] - 50) < 1e-6
    assert abs(res["comm"] - (50 + 40)) < 1e-6  # 1 MiB interpolates to 40 us
    assert abs(res["idle"] - 150) < 1e-6 and res["events"] == 3


def test_daemon_cpu_honours_signal_file(tmp_path):
    from ccbench_b200 import native_build_daemons as nd

    nd.build(only=["cpu"])
    (tmp_path / "daemon_signals").mkdir()
    env = dict(os.environ, PERF_OUTPUT_DIR=str(tmp_path / "perf_files"), DAEMON_CPU_PER_CORE="0")
    p = subprocess.Popen([os.path.join(ROOT, "bin/daemons/daemon_cpu"), "0.05"], cwd=tmp_path, env=env,
                         stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    time.sleep(0.4)
    (tmp_path / "daemon_signals" / "daemon_cpu.signal").write_text("PAUSE\n")
    time.sleep(0.3)
    (tmp_path / "daemon_signals" / "daemon_cpu.signal").write_text("EXIT\n")
    out, _ = p.communicate(timeout=10)
    assert p.returncode == 0 and "stopped" in out
    files = os.listdir(tmp_path / "perf_files")
    assert len(files) == 1 and files[0].startswith("perf_cpu_")
    rows = (tmp_path / "perf_files" / files[0]).read_text().splitlines()
    assert rows[0] == "timestamp_sec,cpu_util,cpu_user,cpu_system,cpu_iowait,mem_used,mem_util"
    stamps = [float(r.split(",")[0]) for r in rows[1:]]
    assert 3 <= len(stamps) <= 12 and max(stamps) < 0.55  # nothing sampled while paused


def test_gpu_daemon_against_a_fake_nvml(tmp_path):
    """The GPU daemon only reads: a stand-in NVML library supplies the readings."""
    from ccbench_b200 import native_build_daemons as nd

    nd.build(only=["gpu_nvidia"])
    src = tmp_path / "fake_nvml.c"
    src.write_text("""
typedef void* dev_t;
int nvmlInit_v2(void){return 0;} int nvmlShutdown(void){return 0;}
int nvmlDeviceGetCount_v2(unsigned*n){*n=2;return 0;}
int nvmlDeviceGetHandleByIndex_v2(unsigned i,dev_t*d){*d=(dev_t)(long)(i+1);return 0;}
int nvmlDeviceGetUtilizationRates(dev_t d,unsigned*u){u[0]=40+(long)d;u[1]=7;return 0;}
int nvmlDeviceGetMemoryInfo(dev_t d,unsigned long long*m){m[0]=1ull<<34;m[1]=0;m[2]=3ull<<20;return 0;}
int nvmlDeviceGetTemperature(dev_t d,int s,unsigned*t){*t=55;return 0;}
int nvmlDeviceGetCurrPcieLinkGeneration(dev_t d,unsigned*g){*g=5;return 0;}
int nvmlDeviceGetCurrPcieLinkWidth(dev_t d,unsigned*w){*w=16;return 0;}
int nvmlDeviceGetClockInfo(dev_t d,int t,unsigned*c){*c=1965;return 0;}
int nvmlDeviceGetPowerUsage(dev_t d,unsigned*p){*p=700000;return 0;}
""")
    lib = tmp_path / "libfake_nvml.so"
    subprocess.run(["gcc", "-shared", "-fPIC", str(src), "-o", str(lib)], check=True)
    (tmp_path / "daemon_signals").mkdir()
    env = dict(os.environ, PERF_OUTPUT_DIR=str(tmp_path / "pf"), DAEMON_NVML_LIB=str(lib))
    p = subprocess.Popen([os.path.join(ROOT, "bin/daemons/daemon_gpu_nvidia"), "0.05"], cwd=tmp_path, env=env)
    time.sleep(0.3)
    (tmp_path / "daemon_signals" / "daemon_gpu_nvidia.signal").write_text("FLUSH_EXIT")
    assert p.wait(timeout=10) == 0
    files = sorted(os.listdir(tmp_path / "pf"))
    assert len(files) == 2 and files[0].startswith("perf_gpu_0_")
    rows = (tmp_path / "pf" / files[1]).read_text().splitlines()
    assert rows[0] == "timestamp_sec,gpu_util,mem_util,mem_used,temperature,pcie_gen,pcie_width,sm_clock,power"
    v = rows[1].split(",")
    assert v[1:] == ["42.000000", "7.000000", "3.000000", "55.000000", "5.000000", "16.000000", "1965.000000", "700.000000"]


def test_run_script_order_of_operations(tmp_path):
    """What the run script must do, in the order that matters: clean stale state, export the
    user's environment before LD_PRELOAD, preload compression : communication : extensions,
    phase 1, clean the rendezvous files, phase 2 with the perf wrapper FIRST, exit with the
    larger of the two return codes."""
    cfg = load_config(CFG)
    cfg.job_choice = "local"
    text = runscript.generate(cfg, ROOT)
    pos = lambda needle, start=0: text.index(needle, start)  # noqa: E731
    clean = pos('rm -f "$BENCH_DIR/nccl_id_file/"*')
    user_env = pos("export CCB_CODEC=")
    preload = pos('LD_PRELOAD="${LD_PRELOAD:-}"')
    comm_lib, ext_lib = pos("libccb_nccl.so"), pos("libnccl_extensions.so")
    phase1 = pos("PHASE1_PRELOAD=")
    between = pos('rm -f "$BENCH_DIR/nccl_id_file/"*', phase1)
    phase2 = pos("Phase 2")
    perf = pos("libperfnccl.so", phase2)
    rejoin = pos("$PHASE1_PRELOAD", perf)
    assert "PERF_GENDATA_TARGETS=" not in text.replace("PERF_GENDATA_TARGETS PERF", "")   # capture runs only
    cfg2 = load_config(CFG)
    cfg2.job_choice, cfg2.benchmark_type = "local", "app_gendata"
    text2 = runscript.generate(cfg2, ROOT)
    assert text2.index("export PERF_GENDATA_TARGETS=") > text2.index("Phase 2")
    gendata = rejoin + 1
    final = pos("if [ $BENCH_RC1 -ge $BENCH_RC2 ]; then exit $BENCH_RC1; else exit $BENCH_RC2; fi")
    assert clean < user_env < preload < comm_lib < ext_lib < phase1 < between < phase2 < perf < rejoin < gendata < final
    assert "perf_files" in text[:clean + 400] and 'rm -rf "$PERF_OUTPUT_DIR"' in text
    assert "daemon_signals" in text and ".signal" in text
    # the benchmark binary's arguments follow the reference's argv
    for phase in (1, 2):
        joined = f" {runscript.bench_args(cfg, phase)} "
        assert (" -m " in joined or " -L " in joined) and " -i " in joined and " -w " in joined and " -d " in joined


@pytest.mark.parametrize("script,produces", [
    ("register_metrics.sh", "bin/libs/validation.so"),
    ("register_job_device_mapper.sh", "bin/libs/libjob_device_mapper.so"),
    ("register_daemons.sh", "bin/daemons/daemon_cpu"),
    ("compile_all.sh", "bin/libs/libnccl_extensions.so"),
])
def test_script_entry_points(script, produces):
    """The shell entry points keep the reference's names and leave its build outputs behind."""
    from pathlib import Path

    root = Path(ROOT)
    r = subprocess.run(["bash", str(root / "scripts" / script)], capture_output=True, text=True, timeout=1200)
    assert r.returncode == 0, r.stdout[-1500:] + r.stderr[-1500:]
    assert (root / produces).exists()


def test_run_script_golden_file():
    """The script for the shipped default configuration, local launcher, byte for byte. When a
    change to the generator is intended, regenerate the golden file with the three lines
    below and review its diff."""
    from pathlib import Path

    cfg = load_config(CFG)
    cfg.job_choice = "local"
    text = runscript.generate(cfg, Path("/opt/ccbench"))
    golden = Path(ROOT) / "tests" / "golden" / "run_benchmark_local_default.sh"
    assert text == golden.read_text(), "generated script differs from tests/golden/run_benchmark_local_default.sh"


def test_configuration_problems_are_named(tmp_path):
    import dataclasses

    cfg = load_config(CFG)
    assert cfg.problems(ROOT) == []
    cfg.arch, cfg.job_choice, cfg.msg_mode, cfg.msg_list = "rccl", "pbs", "list", []
    cfg.comm = dataclasses.replace(cfg.comm, mode=7)
    cfg.perf = dataclasses.replace(cfg.perf, mode=3, source_files=[], source_dirs=[])
    cfg.ds_type, cfg.ds_file = "folder", ""
    cfg.stress_gpu_percent = 250
    text = "\\n".join(cfg.problems(ROOT))
    for needle in ("communication_arch 'rccl'", "job_choice 'pbs'", "non-empty list", "mode 7", "needs source_files", "needs file_path", "250"):
        assert needle in text, (needle, text)
    cfg2 = load_config(CFG)
    cfg2.benchmark_type, cfg2.test_name = "nccl_allscatter", "allscatter"
    assert any("no benchmark named 'allscatter'" in p for p in cfg2.problems())
    cfg3 = load_config(CFG)
    cfg3.benchmark_type, cfg3.app_command, cfg3.gendata_targets = "app_gendata", "", ""
    assert len(cfg3.problems()) == 2
    # the command line refuses such a configuration with the list
    bad = tmp_path / "cfg"
    import shutil

    shutil.copytree(CFG, bad)
    p = bad / "job_config.jsonc"
    p.write_text(p.read_text().replace('"local"', '"pbs"', 1))
    r = subprocess.run([sys.executable, "-m", "ccbench_b200.cli", "--config-dir", str(bad), "gen-script"], capture_output=True, text=True,
                       cwd=ROOT)
    if '"pbs"' in p.read_text():   # the shipped file selects the launcher by that literal
        assert r.returncode == 2 and "job_choice 'pbs'" in r.stderr, r.stderr
