"""Host description as JSON, with the top-level keys of the reference's probe
(.claude/skills/configure-bench/scripts/detect_env.sh:69-410 and the schema it assembles at
:420-510): timestamp, hostname, ccbench_dir, cpu, memory, gpu, cuda, nccl, mpi, ib, network,
ucx, slurm, slurm_allocation, compiler, python, os, modules_loaded, plugin_projects, disk,
datasets, environment, current_config. Added for this framework: per-GPU compute
capability, clocks and NVLink state, peer-access / NVLS-relevant facts, and which of the
repository's own libraries and binaries are built. Read-only: nothing is changed on the
host, no clocks or modes are touched.

    python -m ccbench_b200.utils.detect_env            # prints the JSON
"""
from __future__ import annotations

import glob
import json
import os
import platform
import re
import shutil
import subprocess
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent.parent


def _run(cmd, timeout=10) -> str:
    try:
        return subprocess.run(cmd, capture_output=True, text=True, timeout=timeout).stdout.strip()
    except Exception:
        return ""


def _first_line(cmd) -> str:
    out = _run(cmd)
    return out.splitlines()[0].strip() if out else ""


def _cpu() -> dict:
    model = ""
    try:
        for line in open("/proc/cpuinfo"):
            if line.lower().startswith("model name"):
                model = line.split(":", 1)[1].strip()
                break
    except OSError:
        pass
    nodes = len(glob.glob("/sys/devices/system/node/node[0-9]*")) or 1
    return {"cores": os.cpu_count() or 0, "model": model or "unknown", "architecture": platform.machine(), "numa_nodes": nodes}


def _memory() -> dict:
    vals = {}
    try:
        for line in open("/proc/meminfo"):
            k, v = line.split(":", 1)
            vals[k] = int(v.split()[0])
    except (OSError, ValueError):
        pass
    gb = lambda k: round(vals.get(k, 0) / (1 << 20), 1)
    return {"total_gb": gb("MemTotal"), "available_gb": gb("MemAvailable")}


def _gpus() -> dict:
    devs = []
    if shutil.which("nvidia-smi"):
        q = "index,name,memory.total,driver_version,compute_cap,clocks.max.sm,clocks.max.mem,power.limit,pci.bus_id"
        for line in _run(["nvidia-smi", f"--query-gpu={q}", "--format=csv,noheader"]).splitlines():
            p = [x.strip() for x in line.split(",")]
            if len(p) >= 9:
                devs.append({"index": p[0], "name": p[1], "memory": p[2], "driver": p[3], "compute_capability": p[4],
                             "max_sm_clock": p[5], "max_mem_clock": p[6], "power_limit": p[7], "pci_bus_id": p[8]})
    out = {"nvidia_present": bool(devs), "nvidia_count": len(devs), "nvidia_devices": devs,
           "amd_present": bool(shutil.which("rocminfo")), "amd_count": 0}
    if devs:
        # NVLink: active links of GPU 0 and the topology matrix's verdict between GPU 0 and 1
        links = [l for l in _run(["nvidia-smi", "nvlink", "--status", "-i", "0"]).splitlines() if re.search(r"Link \d+:", l)]
        out["nvlink"] = {"gpu0_links": len(links), "gpu0_link_speeds": sorted({l.split(":", 1)[1].strip() for l in links})}
        topo = _run(["nvidia-smi", "topo", "-m"])
        out["nvswitch_all_to_all"] = bool(re.search(r"\bNV\d+\b", topo)) if topo else None
        out["fabric_manager"] = bool(_run(["pgrep", "-x", "nv-fabricmanager"]))
    return out


def _cuda() -> dict:
    nvcc = shutil.which("nvcc") or ("/usr/local/cuda/bin/nvcc" if os.path.exists("/usr/local/cuda/bin/nvcc") else "")
    version = ""
    if nvcc:
        m = re.search(r"release ([\d.]+)", _run([nvcc, "--version"]))
        version = m.group(1) if m else ""
    home = os.environ.get("CUDA_HOME") or os.environ.get("CUDA_PATH") or (str(Path(nvcc).resolve().parent.parent) if nvcc else "")
    archs = _run([nvcc, "--list-gpu-arch"]).split() if nvcc else []
    return {"found": bool(nvcc), "version": version, "nvcc_path": nvcc, "cuda_home": home,
            "cudart": sorted(glob.glob(os.path.join(home, "lib64", "libcudart.so*")))[:3] if home else [],
            "supports_sm_100a": any(a.endswith("100") or a.endswith("100a") for a in archs),
            "tools": {t: bool(shutil.which(t) or (home and os.path.exists(os.path.join(home, "bin", t)))) for t in ("ncu", "nsys", "compute-sanitizer")}}


def _nccl() -> dict:
    libs = []
    for pat in ("/usr/lib/x86_64-linux-gnu/libnccl.so*", "/usr/local/lib/libnccl.so*", "/usr/lib64/libnccl.so*"):
        libs += glob.glob(pat)
    for d in os.environ.get("LD_LIBRARY_PATH", "").split(":"):
        if d:
            libs += glob.glob(os.path.join(d, "libnccl.so*"))
    version = ""
    for hdr in ("/usr/include/nccl.h", "/usr/local/include/nccl.h", "/usr/local/cuda/include/nccl.h"):
        if os.path.exists(hdr):
            txt = open(hdr, errors="replace").read()
            mm = [re.search(rf"#define NCCL_{k}\s+(\d+)", txt) for k in ("MAJOR", "MINOR", "PATCH")]
            if all(mm):
                version = ".".join(m.group(1) for m in mm)
            break
    torch_nccl = ""
    try:
        import torch

        torch_nccl = ".".join(map(str, torch.cuda.nccl.version())) if hasattr(torch.cuda, "nccl") else ""
    except Exception:
        pass
    base = ROOT / "bin" / "libs" / "base_so_name"
    return {"found": bool(libs or version), "version": version, "library": sorted(set(libs))[0] if libs else "",
            "libraries": sorted(set(libs)), "torch_bundled_version": torch_nccl,
            "recorded_base_library": base.read_text().strip() if base.exists() else ""}


def _mpi() -> dict:
    mpicc, mpirun = shutil.which("mpicc"), shutil.which("mpirun") or shutil.which("mpiexec")
    impl = version = ""
    if mpirun:
        v = _run([mpirun, "--version"])
        impl = "openmpi" if "Open MPI" in v or "OpenRTE" in v else "mpich" if "HYDRA" in v or "MPICH" in v.upper() else \
            "intel" if "Intel" in v else "unknown"
        m = re.search(r"(\d+\.\d+(\.\d+)?)", v)
        version = m.group(1) if m else ""
    return {"found": bool(mpicc or mpirun), "implementation": impl, "version": version, "compiler": mpicc or "",
            "launcher": mpirun or "", "bundled_subset": str(ROOT / "csrc" / "minimpi") if not mpicc else ""}


def _ib() -> dict:
    devs = []
    for d in sorted(glob.glob("/sys/class/infiniband/*")):
        ports = []
        for p in sorted(glob.glob(os.path.join(d, "ports", "*"))):
            rd = lambda f: (open(os.path.join(p, f)).read().strip() if os.path.exists(os.path.join(p, f)) else "")
            ports.append({"port": os.path.basename(p), "state": rd("state"), "rate": rd("rate"), "link_layer": rd("link_layer")})
        devs.append({"name": os.path.basename(d), "ports": ports})
    return {"found": bool(devs), "devices": devs}


def _network() -> dict:
    ifaces = []
    for d in sorted(glob.glob("/sys/class/net/*")):
        name = os.path.basename(d)
        rd = lambda f: (open(os.path.join(d, f)).read().strip() if os.path.exists(os.path.join(d, f)) else "")
        try:
            speed = rd("speed")
        except OSError:
            speed = ""
        ifaces.append({"name": name, "state": rd("operstate"), "speed_mbps": speed, "mtu": rd("mtu")})
    default = ""
    try:
        for line in open("/proc/net/route").read().splitlines()[1:]:
            f = line.split()
            if len(f) > 1 and f[1] == "00000000":
                default = f[0]
                break
    except OSError:
        pass
    return {"interfaces": ifaces, "default_interface": default}


def _ucx() -> dict:
    if not shutil.which("ucx_info"):
        return {"found": False, "transports": []}
    tl = sorted(set(re.findall(r"Transport:\s*(\S+)", _run(["ucx_info", "-d"], timeout=20))))
    return {"found": True, "transports": tl}


def _slurm() -> tuple[dict, dict]:
    found = bool(shutil.which("srun") or shutil.which("sbatch"))
    parts = sorted(set(_run(["sinfo", "-h", "-o", "%P"]).split())) if shutil.which("sinfo") else []
    e = os.environ.get
    alloc = {"job_id": e("SLURM_JOB_ID", ""), "nodelist": e("SLURM_JOB_NODELIST", e("SLURM_NODELIST", "")),
             "nnodes": e("SLURM_NNODES", ""), "ntasks": e("SLURM_NTASKS", ""), "cpus_per_task": e("SLURM_CPUS_PER_TASK", "")}
    return {"found": found, "partitions": parts}, alloc


def _compilers() -> dict:
    ver = lambda exe: (_first_line([exe, "--version"]) if shutil.which(exe) else "")
    return {"gcc": ver("gcc"), "gxx": ver("g++"), "clang": ver("clang"), "cc": shutil.which("cc") or "", "make": bool(shutil.which("make")),
            "ninja": bool(shutil.which("ninja")), "cmake": ver("cmake")}


def _modules() -> tuple[list, dict]:
    loaded = [m for m in os.environ.get("LOADEDMODULES", "").split(":") if m]
    system = "lmod" if os.environ.get("LMOD_CMD") else "environment-modules" if os.environ.get("MODULESHOME") else ""
    return loaded, {"system": system, "modulepath": os.environ.get("MODULEPATH", "")}


def _plugins() -> dict:
    base = ROOT / "plugin_projects"
    ls = lambda p: sorted(x.name for x in p.iterdir() if x.is_dir() and any(x.iterdir())) if p.is_dir() else []
    ext = {}
    for name, patterns in {"sz3": ("libSZ3c.so", "libSZ3.so"), "zfp": ("libzfp.so",), "zccl": ("libZCCL.so",), "dietgpu": ("libdietgpu.so",),
                           "uccl": ("libuccl_p2p.so",)}.items():
        hit = ""
        for d in [*os.environ.get("LD_LIBRARY_PATH", "").split(":"), "/usr/lib/x86_64-linux-gnu", "/usr/local/lib"]:
            for pat in patterns:
                if d and os.path.exists(os.path.join(d, pat)):
                    hit = os.path.join(d, pat)
        ext[name] = hit
    return {"ccl": ls(base / "ccl"), "compression": ls(base / "compression"), "external_libraries": ext}


def _built() -> dict:
    libs = sorted(p.name for p in (ROOT / "bin" / "libs").glob("*.so")) if (ROOT / "bin" / "libs").is_dir() else []
    tests = {arch: sorted(p.name for p in (ROOT / "bin" / arch).iterdir() if p.is_dir()) if (ROOT / "bin" / arch).is_dir() else []
             for arch in ("nccl", "mpi")}
    daemons = sorted(p.name for p in (ROOT / "bin" / "daemons").iterdir()) if (ROOT / "bin" / "daemons").is_dir() else []
    core = ROOT / "ccbench_b200" / "_native" / "libccb.so"
    return {"libccb": core.exists(), "libccb_bytes": core.stat().st_size if core.exists() else 0, "libraries": libs, "benchmarks": tests,
            "daemons": daemons, "run_scripts": sorted(p.name for p in (ROOT / "scripts" / "run").glob("run_benchmark.*")) if (ROOT / "scripts" / "run").is_dir() else []}


def _current_config() -> dict:
    try:
        from ..config.model import load_config

        c = load_config(ROOT / "userconfig" / "config_in_jsonc")
        return {"benchmark_type": c.benchmark_type, "communication_arch": c.arch, "communication_mode": c.comm.mode,
                "compression_mode": c.comp.mode, "perf_mode": c.perf.mode, "job_choice": c.job_choice}
    except Exception as e:  # noqa: BLE001
        return {"error": str(e)}


def detect() -> dict:
    slurm, alloc = _slurm()
    loaded, modsys = _modules()
    disk = shutil.disk_usage(ROOT)
    datasets = sorted(str(p.relative_to(ROOT)) for p in (ROOT / "dataset").rglob("*.f32"))[:50] if (ROOT / "dataset").is_dir() else []
    osname = ""
    try:
        for line in open("/etc/os-release"):
            if line.startswith("PRETTY_NAME="):
                osname = line.split("=", 1)[1].strip().strip('"')
    except OSError:
        osname = platform.platform()
    return {
        "timestamp": time.strftime("%Y-%m-%dT%H:%M:%SZ", time.gmtime()), "hostname": platform.node(), "ccbench_dir": str(ROOT),
        "kernel": platform.release(), "cpu": _cpu(), "memory": _memory(), "gpu": _gpus(), "cuda": _cuda(), "nccl": _nccl(),
        "mpi": _mpi(), "ib": _ib(), "network": _network(), "ucx": _ucx(), "slurm": slurm, "slurm_allocation": alloc,
        "compiler": _compilers(), "python": {"version": platform.python_version(), "command": sys.executable}, "os": osname,
        "modules_loaded": loaded, "module_system": modsys, "plugin_projects": _plugins(),
        "disk": {"ccbench_available_gb": round(disk.free / (1 << 30), 1)}, "datasets": datasets,
        "environment": {"ld_library_path": os.environ.get("LD_LIBRARY_PATH", ""), "cuda_home": os.environ.get("CUDA_HOME", ""),
                        "ld_preload": os.environ.get("LD_PRELOAD", ""), "nccl_debug": os.environ.get("NCCL_DEBUG", "")},
        "current_config": _current_config(), "built": _built(),
        # the old flat keys, kept for callers of the first version of this probe
        "gpus": _gpus()["nvidia_devices"], "cpus": os.cpu_count(),
    }


def main() -> int:
    print(json.dumps(detect(), indent=2))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
