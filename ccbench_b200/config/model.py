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
