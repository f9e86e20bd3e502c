"""Small host utilities: NUMA binding, clock sampler parsing."""
import os

from ccbench_b200.utils import numa
from ccbench_b200.utils.clocks import ClockSampler


def test_cpulist_parsing():
    assert numa._parse_cpulist("0-3,8,10-11\n") == {0, 1, 2, 3, 8, 10, 11}
    assert numa._parse_cpulist("") == set()


def test_topology_table_fallback():
    topo = ("\tGPU0\tGPU1\tNIC0\tCPU Affinity\tNUMA Affinity\tGPU NUMA ID\n"
            "GPU0\t X \tNV18\tSYS\t0-55,112-167\t0\t\tN/A\n"
            "GPU1\tNV18\t X \tSYS\t56-111,168-223\t1\t\tN/A\n")
    assert numa.topo_cpu_affinity(0, topo) == set(range(0, 56)) | set(range(112, 168))
    assert 56 in numa.topo_cpu_affinity(1, topo) and 0 not in numa.topo_cpu_affinity(1, topo)
    assert numa.topo_cpu_affinity(5, topo) == set()


def test_binding_without_a_gpu_changes_nothing():
    before = os.sched_getaffinity(0)
    assert numa.bind_to_gpu_node(0)["node"] == -1
    assert os.sched_getaffinity(0) == before


def test_clock_summary_reads_nvidia_smi_rows(tmp_path):
    s = ClockSampler([0, 1], 100)
    f = tmp_path / "clocks.csv"
    f.write_text("0, 1965, 1965, 412.3, 0x0000000000000004, Not Active, Not Active, Not Active, Active\n"
                 "1, 1950, 1965, 640.0, 0x0000000000000000, Not Active, Not Active, Not Active, Not Active\n"
                 "0, 1935, 1965, 800.1, 0x0000000000000004, Not Active, Not Active, Not Active, Active\n")
    s.file = open(f, "r+")
    out = s.summary()
    assert out["sm_mhz"] == 1950 and out["sm_max_mhz"] == 1965 and out["reasons"] == ["sw_power_cap"] and out["samples"] == 3
    assert s.gpu_index == "0,1"


def test_environment_probe_reports_the_reference_schema():
    """Top-level keys of the reference's probe plus what this framework adds; runs anywhere."""
    import json

    from ccbench_b200.utils import detect_env

    info = detect_env.detect()
    json.dumps(info)   # serialisable
    for key in ("timestamp", "hostname", "ccbench_dir", "cpu", "memory", "gpu", "cuda", "nccl", "mpi", "ib", "network", "ucx", "slurm",
                "slurm_allocation", "compiler", "python", "os", "modules_loaded", "plugin_projects", "disk", "datasets", "environment",
                "current_config", "built"):
        assert key in info, key
    assert info["cpu"]["cores"] >= 1 and info["memory"]["total_gb"] > 0
    assert set(info["gpu"]) >= {"nvidia_present", "nvidia_count", "nvidia_devices", "amd_present", "amd_count"}
    assert set(info["cuda"]) >= {"found", "version", "nvcc_path", "cuda_home"}
    assert set(info["mpi"]) >= {"found", "implementation", "version", "compiler"}
    assert info["current_config"].get("communication_arch") in ("nccl", "mpi", "rccl")
    assert isinstance(info["network"]["interfaces"], list) and info["compiler"]["gcc"]
