"""Reference arm of bench.py: runs the reference's own `bin/nccl/allreduce/allreduce`
benchmark binary, unmodified, in its shipped default configuration (communication
wrapper mode 0: the interposed call goes to bare NCCL,
userconfig/config_in_jsonc/communication_lib_selection.jsonc:25), on the same message
size and data distribution, and prints the same JSON line with "impl": "reference".

The reference's int8 wrapper (plain_nccl_compress, wrapper mode 3) is NOT run: on a
2 x B200 box it hung at 1 MiB (killed by its 120 s limit) and raised "an illegal
memory access was encountered" inside NCCL at 256 MiB
(baseline/reference_mode3_fault_record.txt). Its ring issues an un-grouped ncclSend
followed by ncclRecv on one stream on every rank, and both directions share one
scratch buffer that is freed and re-allocated while earlier asynchronous work may
still use it (plain_nccl_compress.cu:499-534, :557-595, :718-729). Code that faulted
a shared GPU is not run again.

One process per rank is started by torch.distributed.run like the other arm; each
rank execs the reference binary as a child with the rank environment the reference
reads (run_codes/benchmark-core/src/nccl/nccl_utils.c:47-68). The reference times the
call with CUDA events and prints avg/min/max over ranks; the max is used.

Differences forced by the reference, all noted in the printed config:
  * its CLI has no bf16/fp16 type, so the 256 MiB message is fp32 (64 Mi elements);
  * its data come from per-rank files (its DS_TYPE=folder source) filled with the same
    gradient-like distribution;
  * it needs at least 2 ranks.
"""
from __future__ import annotations

import json
import os
import re
import shutil
import subprocess
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref", "CC-Bench")


def _unavailable(why: str):
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)
    return 0


def _ensure_built() -> str | None:
    exe = os.path.join(REF, "bin", "nccl", "allreduce", "allreduce")
    wrap = os.path.join(REF, "bin", "libs", "libnccl_extensions.so")
    if os.path.exists(exe) and os.path.exists(wrap):
        return None
    try:
        subprocess.run(["bash", os.path.join(HERE, "build_reference.sh")], check=True, capture_output=True, timeout=1200)
    except Exception as e:  # noqa: BLE001
        return f"reference build failed: {e}"
    if not (os.path.exists(exe) and os.path.exists(wrap)):
        return "reference build produced no allreduce binary / wrapper"
    return None


def main(args) -> int:
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world < 2:
        return _unavailable("the reference allreduce benchmark needs at least 2 ranks "
                            "(run_codes/benchmarks/nccl/allreduce/allreduce.c:153-158)")
    import torch
    import torch.distributed as dist

    dist.init_process_group("gloo")
    err = [None]
    if rank == 0:
        err[0] = _ensure_built()
    dist.broadcast_object_list(err, src=0)
    if err[0]:
        dist.destroy_process_group()
        return _unavailable(err[0])

    sys.path.insert(0, os.path.dirname(HERE))
    from ccbench_b200.models.workloads import gradient_like

    port = os.environ.get("MASTER_PORT", "0")
    run_dir = f"/tmp/ccb_ref_run_{port}"
    data_dir = os.path.join(run_dir, "data")
    if rank == 0:
        shutil.rmtree(run_dir, ignore_errors=True)
        os.makedirs(os.path.join(run_dir, "nccl_id_file"), exist_ok=True)
        os.makedirs(data_dir, exist_ok=True)
    dist.barrier()
    count = args.bytes // 4
    gradient_like(count, torch.float32, seed=rank).numpy().tofile(os.path.join(data_dir, f"rank_{rank}.bin"))
    dist.barrier()

    exe = os.path.join(REF, "bin", "nccl", "allreduce", "allreduce")
    libs = os.path.join(REF, "bin", "libs")
    env = dict(os.environ)
    env.update({
        "OMPI_COMM_WORLD_RANK": str(rank), "OMPI_COMM_WORLD_SIZE": str(world),
        "OMPI_COMM_WORLD_LOCAL_RANK": str(local_rank), "BENCH_DIR": REF,
        "DS_TYPE": "folder", "DS_SUFFIX": ".bin", "DS_FORMAT": "binary",
        "NCCL_COMPRESS_GROUP": "128", "NCCL_COMPRESS_BITS": "8",
    })
    preload = [os.path.join(libs, "libnccl_extensions.so")]
    compressed = False  # wrapper mode 3 faulted on 2 x B200 and stays off (see the module docstring)
    env["LD_PRELOAD"] = ":".join(preload)

    def run(iters: int, warmup: int, validate: bool):
        if rank == 0:
            for f in os.listdir(os.path.join(run_dir, "nccl_id_file")):
                os.remove(os.path.join(run_dir, "nccl_id_file", f))
            shutil.rmtree(os.path.join(run_dir, "runtime_files"), ignore_errors=True)
            # the reference creates this directory on rank 0 only, racing the other ranks' writes
            os.makedirs(os.path.join(run_dir, "runtime_files", "nccl_agg"), exist_ok=True)
        dist.barrier()
        cmd = [exe, "-L", str(args.bytes), "-i", str(iters), "-w", str(warmup), "-d", "float", "-f", data_dir]
        if validate:
            cmd += ["-v", "-t", "1e30", "-e", "mse"]
        t0 = time.perf_counter()
        p = subprocess.run(cmd, cwd=run_dir, env=env, capture_output=True, text=True, timeout=1500)
        wall = time.perf_counter() - t0
        dist.barrier()
        return p, wall

    p, wall1 = run(args.steps, max(args.warmup, 3), False)
    out = p.stdout
    ok = [p.returncode == 0]
    allok = [None] * world
    dist.all_gather_object(allok, ok[0])
    if not all(allok):
        dist.destroy_process_group()
        return _unavailable("reference benchmark exited non-zero: " + (p.stderr or out)[-300:].replace("\n", " | "))
    line = None
    if rank == 0:
        m = re.search(r"User: avg=\s*([\d.]+) us, min=\s*([\d.]+) us, max=\s*([\d.]+) us", out)
        if not m:
            line = {"impl": "reference", "unavailable": "could not parse the reference output: " + out[-300:].replace("\n", " | ")}
        else:
            t_us = float(m.group(3))
            algbw = args.bytes / (t_us * 1e-6) / 1e9
            line = {
                "metric": "compressed_allreduce_busbw", "value": algbw * 2 * (world - 1) / world * world, "unit": "GB/s",
                "value_definition": "whole-job aggregate: per-GPU bus bandwidth (bytes/t * 2(n-1)/n) summed over the n GPUs; "
                                    "busbw_per_gpu holds the per-GPU figure",
                "busbw_per_gpu": algbw * 2 * (world - 1) / world,
                "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": t_us / 1e3,
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "impl": "reference",
                "config": {"model": "gradient-like buffer: Laplace(0,1e-3) + 0.1% x100 outliers",
                           "message_bytes_per_rank": args.bytes, "global_batch": args.bytes * world,
                           "codec": "int8 group 128 (plain_nccl_compress, wrapper mode 3)" if compressed else "none (bare NCCL, wrapper mode 0)",
                           "algo": "ring, host-driven hops" if compressed else "NCCL", "parallelism": f"dp{world}",
                           "note": "reference CLI has no bf16: fp32 elements, same bytes. The reference's int8 wrapper "
                                   "(mode 3) hung and then faulted on 2 x B200 and is not run; this is its stock mode 0",
                           "timing": "reference's own CUDA events around ncclAllReduce, max over ranks"},
                "algbw": algbw, "ref_definition_bw": 2 * algbw, "gpu_launches": None,
            }
    # deviation: one validated iteration (CPU oracle of the reference)
    pv, _ = run(1, 1, True)
    # end to end: the reference loop uploads the input each iteration (cudaMemcpy from
    # pageable memory) and crosses its TCP barrier; per-iteration wall time is the slope
    # between two iteration counts.
    # 200 extra iterations put seconds between the two runs, so that start-up jitter
    # (NCCL initialisation, data loading) does not swamp the slope; median of three.
    extra = 200
    slopes = []
    for _ in range(3):
        _, wall2 = run(args.steps + extra, max(args.warmup, 3), False)
        slopes.append((wall2 - wall1) / extra)
    slopes.sort()
    if rank == 0 and line and "unavailable" not in line:
        mm = re.search(r"mse: ([\d.eE+-]+)", pv.stdout)
        line["mse"] = float(mm.group(1)) if mm else None
        per_iter = slopes[1] if slopes[1] > 0 else max(slopes)
        if per_iter > 0:
            line["e2e"] = {"value": args.bytes / per_iter / 1e9 * 2 * (world - 1) / world * world, "unit": "GB/s",
                           "busbw_per_gpu": args.bytes / per_iter / 1e9 * 2 * (world - 1) / world,
                           "ms_per_step": per_iter * 1e3, "h2d_bytes_per_step": args.bytes, "d2h_bytes_per_step": 0,
                           "note": f"wall-clock slope between runs of K and K+{extra} iterations of the reference loop, "
                                   "median of three; the loop uploads the input from pageable memory every iteration and "
                                   "reads nothing back"}
    if rank == 0:
        print(json.dumps(line), flush=True)
        shutil.rmtree(run_dir, ignore_errors=True)
    dist.barrier()
    dist.destroy_process_group()
    return 0
