"""Run-script generator: turns the JSONC configuration into
scripts/run/run_benchmark.{sh,srun.sh,mpirun.sh,slurm}.

The generated script has the reference's structure (scripts/build_script.sh:315-859):
clean perf_files / nccl_id_file / signal files, export the data-source and user
environment, locate the base library (findso), build LD_PRELOAD in the order
compression : communication : libnccl_extensions.so, phase 1 (performance round, with
the phase-1 daemons), phase 2 (the perf wrapper prepended, perf-round iteration
counts, gendata variables, phase-2 daemons), exit with the larger return code.
Differences: job_choice "local" starts all ranks with the bundled launcher
(`python -m ccbench_b200.launch`) instead of a single process, and runtime_files/
nccl_agg is created before the ranks start."""
from __future__ import annotations

import os
import shlex
import shutil
from pathlib import Path

from .config.model import BenchConfig

SCRIPT_NAMES = {"slurm": "run_benchmark.slurm", "srun": "run_benchmark.srun.sh", "mpirun": "run_benchmark.mpirun.sh",
                "local": "run_benchmark.sh"}


def launch_command(cfg: BenchConfig, check: bool = True) -> str:
    n = cfg.nprocs
    fwd = "".join(f" -x {k}" for k in cfg.env) if cfg.env else ""
    if cfg.arch == "mpi":
        if cfg.job_choice == "local" and not shutil.which("mpirun"):
            # no MPI on this host: the binaries are linked against the bundled single-host MPI
            # subset, which takes its ranks from the local launcher's environment
            return f"python3 -m ccbench_b200.launch -n {n} --"
        if check and not shutil.which("mpirun"):
            raise RuntimeError("communication_arch=mpi requires mpirun")
        if cfg.job_choice == "srun":
            return f"mpirun -np {n} --hostfile $LSF_HOSTFILE --map-by node" + fwd
        if cfg.job_choice == "mpirun" and cfg.cross_alloc_nodes:
            return f"mpirun --hostfile $CROSS_HOSTFILE -np {n} --map-by node --bind-to none -x LD_LIBRARY_PATH -x LD_PRELOAD" + fwd
        return f"mpirun -np {n}" + fwd
    if cfg.job_choice in ("slurm", "srun"):
        if check and not shutil.which("srun"):
            raise RuntimeError(f"job_choice={cfg.job_choice} requires srun")
        return f"stdbuf -oL srun --nodes={cfg.nodes} --ntasks={n} --ntasks-per-node={cfg.tasks_per_node}"
    if cfg.job_choice == "mpirun":
        if check and not shutil.which("mpirun"):
            raise RuntimeError("job_choice=mpirun requires mpirun")
        if cfg.cross_alloc_nodes:
            return f"mpirun --hostfile $CROSS_HOSTFILE -np {n} --map-by node --bind-to none -x LD_LIBRARY_PATH -x LD_PRELOAD" + fwd
        return f"mpirun -np {n} --bind-to none" + fwd
    if cfg.job_choice == "local":
        return f"python3 -m ccbench_b200.launch -n {n} --" if n > 1 else ""
    raise ValueError(f"unknown job_choice {cfg.job_choice!r}")


def bench_args(cfg: BenchConfig, phase: int) -> str:
    if cfg.msg_mode == "list":
        a = ["-L", ",".join(str(x) for x in cfg.msg_list)]
    else:
        a = ["-m", f"{cfg.msg_min}:{cfg.msg_max}:{cfg.msg_incr}"]
        if cfg.msg_incr_type == "add":
            a.append("-A")
    w, i = (cfg.phase1_warmup, cfg.phase1_measure) if phase == 1 else (cfg.phase2_warmup, cfg.phase2_measure)
    a += ["-i", str(i), "-w", str(w), "-p", cfg.ds_pattern]
    if cfg.validation_enabled:
        a += ["-v", "-e", f'"{cfg.validation_metrics}"']
    if cfg.ds_type in ("file", "folder") and cfg.ds_file:
        a += ["-f", f'"{cfg.ds_file}"']
    a += ["-d", cfg.datatype]
    if cfg.output_csv and cfg.output_csv_path:
        a += ["-c", "-o", f'"{cfg.output_csv_path}"']
    if cfg.output_binary and cfg.output_bin_path:
        a += ["-b", "-B", f'"{cfg.output_bin_path}"']
    return " ".join(a)


def _preload_block(L, name: str, sel) -> None:
    if sel.mode == 0:
        return
    if sel.mode == 1:
        L(f"# {name}: mode 1, preload each prebuilt library")
        for lib in sel.library_paths:
            q = lib if os.path.isabs(lib) else "$BENCH_DIR/" + lib
            L(f'if [ -f "{q}" ]; then LD_PRELOAD="${{LD_PRELOAD:+$LD_PRELOAD:}}{q}"; echo "[bench]   {name}: {q}"; fi')
    else:
        out = sel.output_name
        L(f'if [ -f "$BENCH_DIR/bin/libs/{out}" ]; then')
        L(f'  LD_PRELOAD="${{LD_PRELOAD:+$LD_PRELOAD:}}$BENCH_DIR/bin/libs/{out}"')
        L(f'  echo "[bench]   {name}: $BENCH_DIR/bin/libs/{out}"')
        L("fi")


def _daemon_start(L, daemons, pid_var: str, cfg: BenchConfig) -> None:
    if not cfg.daemons_enabled or not daemons:
        return
    for d in daemons:
        L(f'rm -f "$BENCH_DIR/daemon_signals/daemon_{d}.signal"')
        L(f'if [ -x "$BENCH_DIR/bin/daemons/daemon_{d}" ]; then')
        if cfg.job_choice in ("slurm", "srun"):
            L(f'  srun --overlap --nodes={cfg.nodes} --ntasks={cfg.nodes} --ntasks-per-node=1 "$BENCH_DIR/bin/daemons/daemon_{d}" {cfg.poll_interval} &')
        elif cfg.job_choice == "mpirun" and cfg.nodes > 1:
            L(f'  mpirun -np {cfg.nodes} --map-by node "$BENCH_DIR/bin/daemons/daemon_{d}" {cfg.poll_interval} &')
        else:
            L(f'  "$BENCH_DIR/bin/daemons/daemon_{d}" {cfg.poll_interval} &')
        L(f"  {pid_var}+=($!)")
        L(f'  echo "[bench]   daemon_{d} started (pid $!)"')
        L("else")
        L(f'  echo "[bench]   daemon_{d} not built, skipped"')
        L("fi")


def _daemon_stop(L, daemons, pid_var: str, cfg: BenchConfig) -> None:
    if not cfg.daemons_enabled or not daemons:
        return
    for d in daemons:
        L(f'echo EXIT > "$BENCH_DIR/daemon_signals/daemon_{d}.signal"')
    L(f'for _pid in "${{{pid_var}[@]}}"; do')
    L("  for _i in $(seq 1 100); do kill -0 \"$_pid\" 2>/dev/null || break; sleep 0.1; done")
    L('  kill -0 "$_pid" 2>/dev/null && kill "$_pid" 2>/dev/null')
    L("done")
    for d in daemons:
        L(f'rm -f "$BENCH_DIR/daemon_signals/daemon_{d}.signal"')


def generate(cfg: BenchConfig, bench_dir: str | os.PathLike, check_launcher: bool = False) -> str:
    lines: list[str] = []
    L = lines.append
    launch = launch_command(cfg, check=check_launcher)
    L("#!/usr/bin/env bash")
    if cfg.job_choice == "slurm":
        j = cfg.slurm_job
        for key, flag in (("name", "job-name"), ("output", "output"), ("error", "error"), ("time", "time"),
                          ("partition", "partition"), ("qos", "qos")):
            if j.get(key):
                L(f"#SBATCH --{flag}={j[key]}")
        L(f"#SBATCH --nodes={cfg.nodes}")
        L(f"#SBATCH --ntasks-per-node={cfg.tasks_per_node}")
        r = cfg.resources
        if r.get("cpus_per_task"):
            L(f"#SBATCH --cpus-per-task={r['cpus_per_task']}")
        if r.get("gpus_per_node"):
            L(f"#SBATCH --gres=gpu:{(r.get('gpu_type') + ':') if r.get('gpu_type') else ''}{r['gpus_per_node']}")
        if r.get("memory_gb"):
            L(f"#SBATCH --mem={r['memory_gb']}G")
        if r.get("exclusive"):
            L("#SBATCH --exclusive")
    L("# Generated by ccbench_b200.runscript; edit the JSONC files and regenerate instead of editing this file.")
    L("set -u")
    L(f'BENCH_DIR="${{BENCH_DIR:-{Path(bench_dir).resolve()}}}"')
    L('export BENCH_DIR')
    L('cd "$BENCH_DIR" || exit 1')
    L('export PYTHONPATH="$BENCH_DIR${PYTHONPATH:+:$PYTHONPATH}"')
    L("")
    L("# ---- clean what an earlier run may have left behind")
    L('PERF_OUTPUT_DIR="${PERF_OUTPUT_DIR:-$BENCH_DIR/perf_files}"; export PERF_OUTPUT_DIR')
    L('rm -rf "$PERF_OUTPUT_DIR"; mkdir -p "$PERF_OUTPUT_DIR"')
    L('mkdir -p "$BENCH_DIR/nccl_id_file" "$BENCH_DIR/daemon_signals" "$BENCH_DIR/results" "$BENCH_DIR/runtime_files/nccl_agg"')
    L('rm -f "$BENCH_DIR/nccl_id_file/"* "$BENCH_DIR/runtime_files/nccl_agg/"* "$BENCH_DIR/daemon_signals/"*.signal "$BENCH_DIR/daemon_signals/gendata_done_"*')
    if cfg.output_csv and cfg.output_csv_path:
        L(f'[ "${{CCB_RESUME:-0}}" = 1 ] || rm -f {shlex.quote(cfg.output_csv_path)}')
    L("")
    L("# ---- configuration")
    L(f"BENCHMARK_TYPE={shlex.quote(cfg.benchmark_type)}")
    L(f"ARCH={shlex.quote(cfg.arch)}")
    L(f"TEST_NAME={shlex.quote(cfg.test_name)}")
    L(f"NPROCS={cfg.nprocs}")
    L(f"APP_COMMAND={shlex.quote(cfg.app_command)}")
    L(f"ENV_VAR_NAMES={shlex.quote(' '.join(cfg.env))}")
    L(f"export DS_TYPE={shlex.quote(cfg.ds_type)}")
    L(f"export DS_FORMAT={shlex.quote(cfg.ds_format)}")
    L(f"export DS_SUFFIX={shlex.quote(cfg.ds_suffix)}")
    L(f"export DS_BASE_OFFSET={cfg.ds_base_offset}")
    L(f"export DS_PER_RANK_OFFSET={'true' if cfg.ds_per_rank_offset else 'false'}")
    if cfg.ds_custom_offsets:
        L(f"export DS_CUSTOM_OFFSETS={shlex.quote(','.join(str(int(x)) for x in cfg.ds_custom_offsets))}")
    L(f"export STRESS_CPU_PERCENT={cfg.stress_cpu_percent}")
    L(f"export STRESS_GPU_PERCENT={cfg.stress_gpu_percent}")
    L("# user environment (exported before LD_PRELOAD is set so that the preloaded libraries' own dependencies resolve)")
    for k, v in cfg.env.items():
        L(f"export {k}={shlex.quote(v)}")
    L('export LD_LIBRARY_PATH="$BENCH_DIR/bin/libs${LD_LIBRARY_PATH:+:$LD_LIBRARY_PATH}"')
    if cfg.job_choice == "mpirun" and cfg.cross_alloc_nodes:
        L("")
        L("# ---- hostfile across separate allocations")
        L('CROSS_HOSTFILE="$BENCH_DIR/runtime_files/cross_hostfile"')
        L(': > "$CROSS_HOSTFILE"')
        for h in cfg.cross_alloc_nodes:
            L(f'echo "{h} slots={cfg.tasks_per_node}" >> "$CROSS_HOSTFILE"')
        L("export CROSS_HOSTFILE")
    L("")
    L('echo "============================================"')
    L(f'echo " Benchmark: {cfg.benchmark_type}"')
    L(f'echo " Arch:      {cfg.arch}"')
    L(f'echo " Ranks:     {cfg.nprocs}"')
    L('echo "============================================"')
    L("")
    L('echo "[bench] Step 1: checking the base implementation..."')
    L(f'if [ -x "$BENCH_DIR/bin/{cfg.arch}/findso" ]; then "$BENCH_DIR/bin/{cfg.arch}/findso" || echo "[bench]   findso failed (continuing)"; fi')
    L("")
    L('echo "[bench] Step 2: LD_PRELOAD"')
    L('LD_PRELOAD="${LD_PRELOAD:-}"')
    _preload_block(L, "compression", cfg.comp)
    _preload_block(L, "communication", cfg.comm)
    if cfg.arch in ("nccl", "rccl"):
        L('if [ -f "$BENCH_DIR/bin/libs/libnccl_extensions.so" ]; then LD_PRELOAD="${LD_PRELOAD:+$LD_PRELOAD:}$BENCH_DIR/bin/libs/libnccl_extensions.so"; fi')
    L("PHASE1_PRELOAD=\"$LD_PRELOAD\"")
    L("export LD_PRELOAD")
    L("")
    gdb = f'{cfg.gdb_path or "gdb"} -batch -ex run -ex bt -ex "bt full" --args' if cfg.gdb_enabled else ""
    L(f"GDB_WRAPPER={shlex.quote(gdb)}")
    binary = '"$BENCH_DIR/bin/$ARCH/$TEST_NAME/$TEST_NAME"'

    def run_phase(phase: int) -> None:
        L(f'if [ "$BENCHMARK_TYPE" = app_trace ] || [ "$BENCHMARK_TYPE" = app_gendata ]; then')
        L(f'  echo "[bench] Launching app (phase {phase}): $APP_COMMAND"')
        L('  case "$APP_COMMAND" in')
        L('    *mpirun*) _X=""; for _v in $ENV_VAR_NAMES LD_PRELOAD PERF_OUTPUT_DIR PERF_GENDATA_TARGETS PERF_GENDATA_OUTPUT_DIR PERF_GENDATA_DONE_DIR; do _X="$_X -x $_v"; done')
        L('              eval "${APP_COMMAND/mpirun/mpirun $_X}" ;;')
        L('    *) eval "$APP_COMMAND" ;;')
        L("  esac")
        L("else")
        L(f"  {launch} $GDB_WRAPPER {binary} {bench_args(cfg, phase)}".replace("  $GDB", " $GDB") if launch else f"  $GDB_WRAPPER {binary} {bench_args(cfg, phase)}")
        L("fi")

    L('echo "--- Phase 1: performance round ---"')
    L("PHASE1_DAEMON_PIDS=()")
    _daemon_start(L, cfg.phase1_daemons, "PHASE1_DAEMON_PIDS", cfg)
    run_phase(1)
    L("BENCH_RC1=$?")
    _daemon_stop(L, cfg.phase1_daemons, "PHASE1_DAEMON_PIDS", cfg)
    L("")
    L("# ---- between the phases: stale rendezvous files must not be picked up again")
    L('rm -f "$BENCH_DIR/nccl_id_file/"* "$BENCH_DIR/runtime_files/nccl_agg/"*')
    L("")
    L("BENCH_RC2=0")
    if cfg.perf.mode != 0:
        L('echo "--- Phase 2: breakdown round (perf wrapper first in LD_PRELOAD) ---"')
        L('LD_PRELOAD=""')
        _preload_block(L, "perf", cfg.perf)
        L('LD_PRELOAD="${LD_PRELOAD:+$LD_PRELOAD${PHASE1_PRELOAD:+:}}$PHASE1_PRELOAD"')
        L("export LD_PRELOAD")
        if cfg.benchmark_type == "app_gendata" and cfg.gendata_targets:
            # capture runs only: the perf wrapper dumps the named calls' buffers and ends the run
            L(f"export PERF_GENDATA_TARGETS={shlex.quote(cfg.gendata_targets)}")
            where = cfg.output_bin_path or "gendata"
            where = where if os.path.isabs(where) else "$BENCH_DIR/" + where
            L(f'export PERF_GENDATA_OUTPUT_DIR="${{PERF_GENDATA_OUTPUT_DIR:-{where}}}"')
            L('export PERF_GENDATA_DONE_DIR="${PERF_GENDATA_DONE_DIR:-$BENCH_DIR/daemon_signals}"')
            L('mkdir -p "$PERF_GENDATA_OUTPUT_DIR"')
        L("PHASE2_DAEMON_PIDS=()")
        _daemon_start(L, cfg.phase2_daemons, "PHASE2_DAEMON_PIDS", cfg)
        run_phase(2)
        L("BENCH_RC2=$?")
        _daemon_stop(L, cfg.phase2_daemons, "PHASE2_DAEMON_PIDS", cfg)
    L("")
    L('echo "[bench] phase 1 rc=$BENCH_RC1, phase 2 rc=$BENCH_RC2"')
    L("if [ $BENCH_RC1 -ge $BENCH_RC2 ]; then exit $BENCH_RC1; else exit $BENCH_RC2; fi")
    return "\n".join(lines) + "\n"


def write(cfg: BenchConfig, bench_dir, out_dir=None, check_launcher: bool = False) -> Path:
    out_dir = Path(out_dir or Path(bench_dir) / "scripts" / "run")
    out_dir.mkdir(parents=True, exist_ok=True)
    path = out_dir / SCRIPT_NAMES[cfg.job_choice]
    path.write_text(generate(cfg, bench_dir, check_launcher))
    path.chmod(0o755)
    return path
