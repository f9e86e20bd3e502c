"""Pin the calling process to the CPUs of the NUMA node its GPU hangs off, so that pinned
host buffers allocated afterwards (first touch) and the copy threads are local to the
GPU's PCIe root. Process-level CPU affinity only; nothing on the GPU is changed."""
from __future__ import annotations

import os


def _parse_cpulist(text: str) -> set[int]:
    cpus: set[int] = set()
    for part in text.strip().split(","):
        if not part:
            continue
        if "-" in part:
            a, b = part.split("-")
            cpus.update(range(int(a), int(b) + 1))
        else:
            cpus.add(int(part))
    return cpus


def gpu_numa_node(device_index: int) -> int:
    """NUMA node of a CUDA device from sysfs, or -1 when the host does not say."""
    import torch

    p = torch.cuda.get_device_properties(device_index)
    bdf = f"{getattr(p, 'pci_domain_id', 0):04x}:{p.pci_bus_id:02x}:{p.pci_device_id:02x}.0"
    try:
        with open(f"/sys/bus/pci/devices/{bdf}/numa_node") as f:
            return int(f.read().strip())
    except (OSError, ValueError, AttributeError):
        return -1


def topo_cpu_affinity(device_index: int, topo_text: str | None = None) -> set[int]:
    """CPU affinity of a GPU as `nvidia-smi topo -m` reports it (read-only query): the
    fallback for hosts (containers) whose sysfs does not tell the NUMA node."""
    import re
    import shutil
    import subprocess

    if topo_text is None:
        exe = shutil.which("nvidia-smi")
        if not exe:
            return set()
        try:
            topo_text = subprocess.run([exe, "topo", "-m"], capture_output=True, text=True, timeout=20).stdout
        except Exception:
            return set()
    topo_text = re.sub(r"\x1b\[[0-9;]*m", "", topo_text)
    for line in topo_text.splitlines():
        cells = line.split()
        if cells and cells[0] == f"GPU{device_index}":
            for c in cells[1:]:
                if re.fullmatch(r"\d+(-\d+)?(,\d+(-\d+)?)*", c) and ("-" in c or "," in c):
                    return _parse_cpulist(c)
    return set()


def bind_to_gpu_node(device_index: int) -> dict:
    """Returns what was done: {"node": n, "cpus": count}, {"node": -1, "cpus": count,
    "source": "nvidia-smi topo"} when only the topology table knew, or {"node": -1}."""
    try:
        node = gpu_numa_node(device_index)
        if node < 0:
            cpus = topo_cpu_affinity(device_index)
            allowed = os.sched_getaffinity(0) & cpus
            if not allowed or allowed == os.sched_getaffinity(0):
                return {"node": -1}
            os.sched_setaffinity(0, allowed)
            return {"node": -1, "cpus": len(allowed), "source": "nvidia-smi topo"}
        with open(f"/sys/devices/system/node/node{node}/cpulist") as f:
            cpus = _parse_cpulist(f.read())
        allowed = os.sched_getaffinity(0) & cpus
        if not allowed:
            return {"node": node, "cpus": 0}
        os.sched_setaffinity(0, allowed)
        return {"node": node, "cpus": len(allowed)}
    except Exception:  # a host that hides sysfs or forbids affinity changes: carry on unbound
        return {"node": -1}
