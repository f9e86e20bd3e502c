"""The headline collective through the product's front door: the NCCL all-reduce benchmark
driver (`bin/nccl/allreduce/allreduce`, the same argv as the reference's
run_codes/benchmarks/nccl/allreduce/allreduce.c:71-146) run unchanged under
`LD_PRELOAD=libccb_nccl.so:libnccl_extensions.so`, so that its plain `ncclAllReduce`
lands in the fused kernel. Every rank of an initialised torch.distributed job starts one
driver process on its own GPU; the driver times each call with CUDA events and reports
the maximum over its ranks, which is what `run()` returns next to the deviation metrics
of one validated iteration (the driver's CPU oracle, summed in float64).
"""
from __future__ import annotations

import os
import re
import shutil
import subprocess
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent.parent
_DTYPE_FLAG = {"bf16": "bfloat16", "f16": "half", "f32": "float"}


def run(x, *, rank: int, world: int, local_rank: int, nbytes: int, dtype: str, codec: str, algo: str, steps: int,
        warmup: int, nvls: bool = False, validate: bool = True) -> dict | None:
    """`x` is this rank's input tensor (its bytes become the driver's per-rank data file).
    Returns a dict on rank 0, None elsewhere."""
    import torch
    import torch.distributed as dist

    from ..native_build import build_c_targets

    exe = ROOT / "bin" / "nccl" / "allreduce" / "allreduce"
    libs = ROOT / "bin" / "libs"
    if rank == 0:
        if not (exe.exists() and (libs / "libccb_nccl.so").exists()):
            build_c_targets()
        from ..wrapper_build import register_metrics

        register_metrics()   # bin/libs/validation.so from the current metric sources
    dist.barrier()
    port = os.environ.get("MASTER_PORT", "0")
    run_dir = Path(f"/tmp/ccb_via_{port}")
    data_dir = run_dir / "data"
    if rank == 0:
        shutil.rmtree(run_dir, ignore_errors=True)
        (run_dir / "nccl_id_file").mkdir(parents=True)
        data_dir.mkdir()
    dist.barrier()
    raw = x.detach().cpu().contiguous()
    (raw.view(torch.int16) if raw.element_size() == 2 else raw).numpy().tofile(data_dir / f"rank_{rank}.bin")
    dist.barrier()

    env = dict(os.environ)
    env.update({
        "OMPI_COMM_WORLD_RANK": str(rank), "OMPI_COMM_WORLD_SIZE": str(world), "OMPI_COMM_WORLD_LOCAL_RANK": str(local_rank),
        "BENCH_DIR": str(ROOT), "DS_TYPE": "folder", "DS_SUFFIX": ".bin", "DS_FORMAT": "binary",
        "CCB_CODEC": codec, "CCB_ALGO": algo if algo in ("twoshot", "oneshot", "ring", "tree", "nvls") else "auto",
        "LD_PRELOAD": f"{libs / 'libccb_nccl.so'}:{libs / 'libnccl_extensions.so'}",
    })
    if nvls:
        env["CCB_NVLS"] = "1"
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):  # the driver reads the launcher chain, not torch's names
        env.pop(k, None)

    def once(iters: int, warm: int, check: bool):
        if rank == 0:
            for f in (run_dir / "nccl_id_file").iterdir():
                f.unlink()
            shutil.rmtree(run_dir / "runtime_files", ignore_errors=True)
            (run_dir / "runtime_files" / "nccl_agg").mkdir(parents=True)
        dist.barrier()
        cmd = [str(exe), "-L", str(nbytes), "-i", str(iters), "-w", str(warm), "-d", _DTYPE_FLAG[dtype], "-f", str(data_dir)]
        if check:
            cmd += ["-v", "-t", "1e30", "-e", "rel_l2,max_abs_err,psnr"]
        p = subprocess.run(cmd, cwd=run_dir, env=env, capture_output=True, text=True, timeout=1500)
        ok = [None] * world
        dist.all_gather_object(ok, p.returncode == 0)
        return p, all(ok)

    p, ok = once(steps, max(warmup, 3), False)
    out = None
    if rank == 0:
        m = re.search(r"User: avg=\s*([\d.]+) us, min=\s*([\d.]+) us, max=\s*([\d.]+) us", p.stdout)
        if not ok or not m:
            out = {"error": ((p.stderr or "") + p.stdout)[-400:].replace("\n", " | ")}
        else:
            t_us = float(m.group(3))
            out = {"ms_per_step": t_us / 1e3, "avg_us": float(m.group(1)),
                   "busbw_per_gpu": nbytes / (t_us * 1e-6) / 1e9 * 2 * (world - 1) / world,
                   "command": f"LD_PRELOAD=libccb_nccl.so:libnccl_extensions.so bin/nccl/allreduce/allreduce -L {nbytes} "
                              f"-i {steps} -w {max(warmup, 3)} -d {_DTYPE_FLAG[dtype]} -f <per-rank files>",
                   "timing": "the driver's CUDA events around ncclAllReduce, max over ranks"}
    if validate and ok:
        pv, okv = once(1, 1, True)
        if rank == 0 and out is not None and "error" not in out:
            out["report"] = [ln.strip() for ln in pv.stdout.splitlines() if re.search(r"Correct:|rel_l2|max_abs_err|psnr", ln)]
            for name in ("rel_l2", "max_abs_err", "psnr"):
                mm = re.search(name + r":\s*([-+\d.eE]+|inf|nan)", pv.stdout)
                out[name] = float(mm.group(1)) if mm else None
    dist.barrier()
    if rank == 0:
        shutil.rmtree(run_dir, ignore_errors=True)
    return out
