"""The eight JSONC configuration files as one object, with the same keys, defaults
and derived values as the reference's generator (scripts/build_script.sh:45-214,
246-303): benchmark_type "<arch>_<test>", wrapper selection files with modes 0-3,
daemon lists, validation metrics, environment map, message sizes, iteration counts."""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any

from .jsonc import load as jsonc_load

FILES = ["bench_basic_config", "job_config", "communication_lib_selection", "compression_kernel_selection",
         "perf_kernel_selection", "daemon_config", "deviation_config", "environment_variables"]

DATATYPES = {"MPI_FLOAT": "float", "MPI_DOUBLE": "double", "MPI_INT": "int", "MPI_CHAR": "char",
             "float": "float", "double": "double", "int": "int", "char": "char"}


@dataclass
class WrapperSel:
    mode: int = 0
    library_paths: list = field(default_factory=list)
    source_files: list = field(default_factory=list)
    source_dirs: list = field(default_factory=list)
    include_files: list = field(default_factory=list)
    include_dirs: list = field(default_factory=list)
    libraries: list = field(default_factory=list)
    output_name: str = ""

    @classmethod
    def from_dict(cls, d: dict) -> "WrapperSel":
        return cls(int(d.get("mode", 0)), list(d.get("library_paths", [])), list(d.get("source_files", [])),
                   list(d.get("source_dirs", [])), list(d.get("include_files", [])), list(d.get("include_dirs", [])),
                   list(d.get("libraries", [])), d.get("output_name", ""))


def _csv_list(s) -> list:
    if isinstance(s, (list, tuple)):
        return [str(x).strip() for x in s if str(x).strip()]
    return [x.strip() for x in str(s or "").split(",") if x.strip()]


@dataclass
class BenchConfig:
    raw: dict
    benchmark_type: str
    arch: str
    test_name: str
    app_command: str
    gendata_targets: str            # PERF_GENDATA_TARGETS form: "op:occ,occ;op:occ"
    gdb_enabled: bool
    gdb_path: str
    snapshot_level: str
    snapshot_dir: str
    ds_type: str
    ds_file: str
    ds_pattern: str
    ds_format: str
    ds_suffix: str
    ds_base_offset: int
    ds_per_rank_offset: bool
    ds_custom_offsets: list
    output_csv: bool
    output_csv_path: str
    output_binary: bool
    output_bin_path: str
    datatype: str
    phase1_warmup: int
    phase1_measure: int
    phase2_warmup: int
    phase2_measure: int
    msg_mode: str
    msg_min: int
    msg_max: int
    msg_incr: int
    msg_incr_type: str
    msg_list: list
    job_choice: str
    cross_alloc_nodes: list
    slurm_job: dict
    nodes: int
    tasks_per_node: int
    resources: dict
    comm: WrapperSel
    comp: WrapperSel
    perf: WrapperSel
    selected_daemons: list
    daemons_enabled: bool
    phase1_daemons: list
    phase2_daemons: list
    poll_interval: float
    stress_cpu_percent: int
    stress_gpu_percent: int
    validation_enabled: bool
    validation_metrics: str
    env: dict

    @property
    def nprocs(self) -> int:
        return self.nodes * self.tasks_per_node

    @property
    def is_app(self) -> bool:
        return self.benchmark_type in ("app_trace", "app_gendata")

    def problems(self, root: str | os.PathLike | None = None) -> list[str]:
        """What is wrong with this configuration, in the user's words: one line per problem,
        empty when it can be turned into a run script. `root` enables the checks that look
        at the repository (benchmark binaries known, prebuilt libraries present)."""
        out: list[str] = []
        tests = ("allreduce", "allgather", "allgatherv", "alltoall", "bcast", "gather", "overlap", "pingpong", "reduce",
                 "reducescatter", "scatter", "scatterv")
        if self.arch not in ("mpi", "nccl"):
            out.append(f"communication_arch {self.arch!r}: expected mpi or nccl (rccl has no benchmarks on this hardware)")
        if not self.is_app and self.test_name not in tests:
            out.append(f"benchmark_type {self.benchmark_type!r}: no benchmark named {self.test_name!r}; known: " + ", ".join(tests))
        if self.is_app and not self.app_command.strip():
            out.append(f"benchmark_type {self.benchmark_type} needs app_command")
        if self.benchmark_type == "app_gendata" and not self.gendata_targets:
            out.append("benchmark_type app_gendata needs gendata_capture.targets with at least one occurrence")
        if self.job_choice not in ("slurm", "srun", "mpirun", "local"):
            out.append(f"job_choice {self.job_choice!r}: expected slurm, srun, mpirun or local")
        if self.nodes < 1 or self.tasks_per_node < 1:
            out.append("slurm.resources.nodes and tasks_per_node must be at least 1")
        for kind, sel in (("communication", self.comm), ("compression", self.comp), ("perf", self.perf)):
            if sel.mode not in (0, 1, 2, 3):
                out.append(f"{kind} selection: mode {sel.mode} is not one of 0 (off), 1 (prebuilt), 2 (build + link), 3 (build)")
            elif sel.mode == 1 and not sel.library_paths:
                out.append(f"{kind} selection: mode 1 needs library_paths")
            elif sel.mode in (2, 3) and not (sel.source_files or sel.source_dirs):
                out.append(f"{kind} selection: mode {sel.mode} needs source_files or source_dirs")
            elif sel.mode in (2, 3) and not sel.output_name:
                out.append(f"{kind} selection: mode {sel.mode} needs output_name")
            if root is not None and sel.mode == 1:
                for lib in sel.library_paths:
                    p = Path(lib) if os.path.isabs(lib) else Path(root) / lib
                    if not p.exists() and not str(lib).startswith("bin/libs/"):
                        out.append(f"{kind} selection: library {lib} does not exist")
        if self.msg_mode not in ("range", "list"):
            out.append(f"message_sizes.mode {self.msg_mode!r}: expected range or list")
        elif self.msg_mode == "list" and not self.msg_list:
            out.append("message_sizes.mode list needs a non-empty list")
        elif self.msg_mode == "range":
            if self.msg_min < 1 or self.msg_max < self.msg_min:
                out.append(f"message_sizes: min {self.msg_min} and max {self.msg_max} do not make a range")
            if self.msg_incr_type not in ("multiply", "add"):
                out.append(f"message_sizes.increment_type {self.msg_incr_type!r}: expected multiply or add")
            elif self.msg_incr < (2 if self.msg_incr_type == "multiply" else 1):
                out.append(f"message_sizes.increment {self.msg_incr} never reaches max")
        if self.ds_type not in ("pattern", "file", "folder"):
            out.append(f"data_source.type {self.ds_type!r}: expected pattern, file or folder")
        elif self.ds_type in ("file", "folder") and not self.ds_file:
            out.append(f"data_source.type {self.ds_type} needs file_path")
        if min(self.phase1_measure, self.phase2_measure) < 1 or min(self.phase1_warmup, self.phase2_warmup) < 0:
            out.append("iterations: measurement counts must be at least 1 and warm-up counts not negative")
        for pct, name in ((self.stress_cpu_percent, "cpu_percent"), (self.stress_gpu_percent, "gpu_percent")):
            if not 0 <= pct <= 100:
                out.append(f"daemon stress.{name} {pct}: expected 0..100")
        return out


def load_config(config_dir: str | os.PathLike) -> BenchConfig:
    d = Path(config_dir)
    raw: dict[str, Any] = {}
    for name in FILES:
        p = d / f"{name}.jsonc"
        raw[name] = jsonc_load(p) if p.exists() else {}
    b, j = raw["bench_basic_config"], raw["job_config"]
    btype = b.get("benchmark_type", "nccl_allreduce")
    arch = b.get("communication_arch", btype.split("_", 1)[0] if "_" in btype else "nccl")
    ds = b.get("data_source", {})
    off = ds.get("offset_config", {})
    out = b.get("output", {})
    it = b.get("iterations", {})
    ms = b.get("message_sizes", {})
    targets = []
    for t in b.get("gendata_capture", {}).get("targets", []):
        occ = ",".join(str(int(o)) for o in t.get("occurrence", []))
        if occ:
            targets.append(f"{t.get('operation', 'all')}:{occ}")
    slurm = j.get("slurm", {})
    res = slurm.get("resources", {})
    dm = raw["daemon_config"]
    perf = dm.get("performance", {})
    val = raw["deviation_config"].get("validation", {})
    dt = b.get("mpi_operation", {}).get("datatype", "MPI_DOUBLE")
    return BenchConfig(
        raw=raw, benchmark_type=btype, arch=arch, test_name=btype.split("_", 1)[1] if "_" in btype else btype,
        app_command=b.get("app_command", ""), gendata_targets=";".join(targets),
        gdb_enabled=bool(b.get("debug", {}).get("gdb_enabled", False)), gdb_path=b.get("debug", {}).get("gdb_path", "gdb"),
        snapshot_level=b.get("snapshot", {}).get("level", "off"), snapshot_dir=b.get("snapshot", {}).get("save_dir", "env_saves"),
        ds_type=ds.get("type", "pattern"), ds_file=ds.get("file_path", ""), ds_pattern=ds.get("pattern_type", "rank_linear"),
        ds_format=ds.get("file_format", "binary"), ds_suffix=ds.get("file_suffix", ""),
        ds_base_offset=int(off.get("base_offset", 0)), ds_per_rank_offset=bool(off.get("per_rank_offset", True)),
        ds_custom_offsets=list(off.get("custom_offsets", [])),
        output_csv=bool(out.get("csv", False)), output_csv_path=out.get("csv_path", ""),
        output_binary=bool(out.get("binary", False)), output_bin_path=out.get("bin_path", ""),
        datatype=DATATYPES.get(dt, "double"),
        phase1_warmup=int(it.get("performance", {}).get("warmup", 10)), phase1_measure=int(it.get("performance", {}).get("measurement", 100)),
        phase2_warmup=int(it.get("perf_round", {}).get("warmup", 3)), phase2_measure=int(it.get("perf_round", {}).get("measurement", 5)),
        msg_mode=ms.get("mode", "range"), msg_min=int(ms.get("min", 1)), msg_max=int(ms.get("max", 65536)),
        msg_incr=int(ms.get("increment", 2)), msg_incr_type=ms.get("increment_type", "multiply"),
        msg_list=[int(x) for x in ms.get("list", [])],
        job_choice=j.get("job_choice", "local"), cross_alloc_nodes=list(j.get("cross_alloc_nodes", [])),
        slurm_job=dict(slurm.get("job", {})), nodes=int(res.get("nodes", 1)), tasks_per_node=int(res.get("tasks_per_node", 1)),
        resources=dict(res),
        comm=WrapperSel.from_dict(raw["communication_lib_selection"]),
        comp=WrapperSel.from_dict(raw["compression_kernel_selection"]),
        perf=WrapperSel.from_dict(raw["perf_kernel_selection"]),
        selected_daemons=_csv_list(dm.get("selected_daemons", "")), daemons_enabled=bool(perf.get("enabled", False)),
        phase1_daemons=_csv_list(perf.get("phase1_daemons", "")), phase2_daemons=_csv_list(perf.get("phase2_daemons", "")),
        poll_interval=float(perf.get("poll_interval_sec", 1.0)),
        stress_cpu_percent=int(dm.get("stress", {}).get("cpu_percent", 0)), stress_gpu_percent=int(dm.get("stress", {}).get("gpu_percent", 0)),
        validation_enabled=bool(val.get("enabled", False)), validation_metrics=",".join(_csv_list(val.get("selected_metrics", ""))),
        env={str(k): str(v) for k, v in raw["environment_variables"].items()},
    )
