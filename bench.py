#!/usr/bin/env python
"""Headline benchmark: compressed AllReduce bus bandwidth on gradient-like data.

    python bench.py --gpus N --steps K --warmup W            (N = 1)
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N \
        --master-addr 127.0.0.1 --master-port P bench.py --gpus N --steps K --warmup W

One "step" is one AllReduce(sum) of a 256 MiB bf16 buffer per rank (Laplace(0, 1e-3)
values with 0.1 % of the entries multiplied by 100), compressed to int8 with one
absmax/127 scale per 128 values, done by ONE fused kernel per rank (two-shot over
NVSwitch peer memory). The reported value is nccl-tests bus bandwidth
(algbw * 2(n-1)/n, algbw = message bytes / time) with the time taken on the device
and the maximum over ranks; at N = 1 there is no bus, so the value is algbw of the
local quantise/dequantise round trip the kernel still performs.

`--impl reference` runs the reference's own allreduce benchmark binary (built unmodified
under baseline/_ref) in its stock configuration, wrapper mode 0 = bare NCCL on the same
bytes, and prints the same line; its int8 wrapper (mode 3) hung and then faulted on
2 x B200 and is not run (baseline/reference_mode3_fault_record.txt).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--bytes", type=int, default=256 << 20, help="message bytes per rank")
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "f32", "f16"])
    ap.add_argument("--codec", default="int8", choices=["int8", "fp8", "none", "int8_g256", "int4"])
    ap.add_argument("--algo", default="tune", choices=["tune", "auto", "twoshot", "oneshot", "ring", "tree", "nvls"],
                    help="tune: time two-shot and ring on this message before the warm-up; ring (one "
                         "requantisation per hop) is kept only when it is more than 15 %% faster")
    ap.add_argument("--error-feedback", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-call-overlap", action="store_true", help="time the calls strictly one after the other")
    ap.add_argument("--via", default="api", choices=["api", "interposer"],
                    help="interposer: also run the same collective through the NCCL benchmark driver under "
                         "LD_PRELOAD=libccb_nccl.so and report its device time beside the direct-API time")
    return ap.parse_args()


def main():
    args = parse()
    if args.impl == "reference":
        from baseline.run_reference import main as ref_main

        return ref_main(args)

    import torch
    import torch.distributed as dist

    from ccbench_b200 import Communicator
    from ccbench_b200.comm import launch_count
    from ccbench_b200.models.workloads import gradient_like
    from ccbench_b200.ops.codecs import wire_ratio
    from ccbench_b200.utils.clocks import ClockSampler

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run for --gpus > 1")
    torch.cuda.set_device(local_rank)
    # host buffers and copy threads next to this GPU's PCIe root (matters for the end-to-end number)
    from ccbench_b200.utils.numa import bind_to_gpu_node
    numa = bind_to_gpu_node(local_rank)
    dev = torch.device("cuda", local_rank)
    pipelined = "on"
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        # Pre-flight of the warp-specialised kernel on a scratch communicator with a short
        # limit on its device-side waits: if it does not complete or does not add up on this
        # job shape, the timed communicator runs the plain two-shot kernel instead. A wait
        # that runs out returns an error status; nothing hangs.
        scratch = Communicator.from_torch_distributed(arena_bytes=256 << 20)
        scratch.set_timeout_ms(3000)
        scratch.set_pipeline(2)
        px = gradient_like(32 << 20, torch.bfloat16, seed=100 + rank, device=dev)   # 64 MiB: several waves per CTA
        py = torch.empty_like(px)
        want = px.float().clone()
        dist.all_reduce(want)
        ok = 1
        try:
            scratch.all_reduce(px, py, codec="int8", algo="twoshot")
            torch.cuda.synchronize()
            rel = ((py.float() - want).norm() / want.norm()).item()
            if scratch.status()[0] != 0 or not rel < 0.1:
                ok = 0
        except Exception:
            ok = 0
        flag = torch.tensor([ok], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        # the same for consecutive calls that overlap tail and head (alternating outputs)
        ok2 = int(flag.item())
        if ok2:
            try:
                py2 = torch.empty_like(px)
                scratch.set_call_overlap(True)
                for k in range(6):
                    scratch.all_reduce(px, (py, py2)[k & 1], codec="int8", algo="twoshot")
                torch.cuda.synchronize()
                for out in (py, py2):
                    rel = ((out.float() - want).norm() / want.norm()).item()
                    if scratch.status()[0] != 0 or not rel < 0.1:
                        ok2 = 0
                del py2
            except Exception:
                ok2 = 0
        flag2 = torch.tensor([ok2], device=dev)
        dist.all_reduce(flag2, op=dist.ReduceOp.MIN)
        scratch.close()
        del px, py, want
        comm = Communicator.from_torch_distributed(nvls=(args.algo == "nvls"))
        if int(flag.item()) == 0:
            comm.set_pipeline(0)
            pipelined = "off: its pre-flight on a scratch communicator failed"
        overlap_ok = int(flag2.item()) == 1 and not args.error_feedback and not args.no_call_overlap
    else:
        comm = Communicator.create(0, 1, f"bench{os.getpid()}")
        overlap_ok = False
        pipelined = "not used with one rank"

    dtype = {"bf16": torch.bfloat16, "f32": torch.float32, "f16": torch.float16}[args.dtype]
    count = args.bytes // torch.empty((), dtype=dtype).element_size()
    x = gradient_like(count, dtype, seed=rank, device=dev)
    y = torch.empty_like(x)
    # Consecutive timed calls write alternating output buffers (as the buckets of a gradient
    # synchronisation do), which lets call k + 1 start on the SMs that call k's CTAs have left.
    ys = [y, torch.empty_like(x)] if overlap_ok else [y]
    ncalls = [0]
    ef = torch.zeros(count, device=dev) if args.error_feedback else None

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    requested = args.algo
    tuning = None
    if args.algo == "tune":
        if world > 1:
            # the exact sum, for the error of each candidate
            exact0 = x.float().clone()
            dist.all_reduce(exact0)
            args.algo, tuning = comm.tune_all_reduce(x, y, codec=args.codec, algos=("twoshot", "ring"), reference=exact0,
                                                      prefer="twoshot", margin=0.15, report=True)
            del exact0
        else:
            args.algo = "twoshot"

    def step():
        comm.all_reduce(x, ys[ncalls[0] % len(ys)], codec=args.codec, algo=args.algo, error_feedback=ef)
        ncalls[0] += 1

    def timed_loop():
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        a.record()
        for _ in range(args.steps):
            step()
        b.record()
        barrier()
        tt = torch.tensor([a.elapsed_time(b)], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        return tt.item() / args.steps

    # Warm up for at least W steps AND about a second, so that the clock sampler (one
    # nvidia-smi sample per 100 ms) sees the GPU under the same load as the timed steps.
    # Rank 0 samples every GPU of the job with one nvidia-smi process and waits for its
    # first line before any rank goes on.
    sampler = ClockSampler(list(range(world)) if rank == 0 else 0, 100)
    if rank == 0:
        sampler.__enter__()
        sampler.wait_first()
    barrier()
    t_w = time.perf_counter()
    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    per = (time.perf_counter() - t_w) / max(args.warmup, 3)
    extra = torch.tensor([min(20000, int(1.2 / max(per, 1e-6)) + 1)], device=dev)
    if world > 1:
        dist.all_reduce(extra, op=dist.ReduceOp.MAX)  # every rank must issue the same number of calls
    for i in range(int(extra.item())):
        step()
        if i % 16 == 15:
            torch.cuda.synchronize()
    barrier()
    rc, words = comm.status()
    if rc != 0:
        raise SystemExit(f"communicator error during warm-up: {words}")

    # ---- the same K steps with every call waiting for the whole call before it ----
    serialised_ms = None
    if overlap_ok and args.algo == "twoshot":
        serialised_ms = timed_loop()
        comm.set_call_overlap(True)
        for _ in range(4):
            step()
    call_overlap = ("on: consecutive calls write alternating output buffers and the first CTAs of call k+1 start on the SMs "
                    "that call k's CTAs have left (Communicator.set_call_overlap); serialised_ms_per_step is the same loop "
                    "without it") if serialised_ms is not None else "off"

    # ---- device-timed region -------------------------------------------------
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    l0 = launch_count()
    barrier()
    start.record()
    for _ in range(args.steps):
        step()
    stop.record()
    barrier()
    sampler.__exit__(None, None, None)
    clk = sampler
    launches = launch_count() - l0
    rc, words = comm.status()
    failed = torch.tensor([1 if rc != 0 else 0], device=dev)
    if world > 1:
        dist.all_reduce(failed, op=dist.ReduceOp.MAX)
    ms = start.elapsed_time(stop)
    t = torch.tensor([ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_per_step = t.item() / args.steps
    if int(failed.item()):
        if serialised_ms is None:
            raise SystemExit(f"communicator error in the timed region: {words}")
        # The loop of overlapping calls did not complete on some rank (a device-side wait gave
        # up; nothing hangs). The serialised loop of the same K steps, timed just before, is
        # the measurement; the rest of the run uses a fresh communicator without overlap.
        ms_per_step = serialised_ms
        call_overlap = f"off: the loop of overlapping calls did not complete (status {words}); the value is the serialised loop"
        try:
            comm.close()
        except Exception:
            pass
        comm = Communicator.from_torch_distributed(nvls=(args.algo == "nvls"))
        if pipelined != "on":
            comm.set_pipeline(0)
        ys = [y]
        for _ in range(3):
            step()
        torch.cuda.synchronize()
    clocks = clk.summary()

    # ---- accuracy of the last result against the exact fp32 sum ----------------
    exact = x.float().clone()
    if world > 1:
        dist.all_reduce(exact)
    comm.set_call_overlap(False)
    rel_l2 = max(((out.float() - exact).norm() / exact.norm()).item() for out in ys)
    del exact
    if len(ys) > 1:
        ys.pop()

    # ---- end to end: pinned host input -> H2D -> AllReduce -> D2H of a sample ----
    e2e = None
    if not args.no_e2e:
        hx = torch.empty(count, dtype=dtype).pin_memory()
        hx.copy_(x)
        # the whole result comes back every step, into two pinned buffers in turn
        hy = [torch.empty(count, dtype=dtype).pin_memory(), torch.empty(count, dtype=dtype).pin_memory()]
        copy_stream, back_stream = torch.cuda.Stream(), torch.cuda.Stream()
        xin = [torch.empty_like(x), torch.empty_like(x)]
        yout = [y, torch.empty_like(x)]
        ready = [torch.cuda.Event(), torch.cuda.Event()]
        freed = [torch.cuda.Event(), torch.cuda.Event()]
        done = [torch.cuda.Event(), torch.cuda.Event()]
        copied = [torch.cuda.Event(), torch.cuda.Event()]

        hm = [torch.empty(1, dtype=torch.float32).pin_memory(), torch.empty(1, dtype=torch.float32).pin_memory()]

        def e2e_loop(k, duplex=True, full=True):
            # Three stages in flight: the upload of step i+1, the collective of step i and the
            # read-back of step i-1 (two device buffers each way). The host waits for the
            # result of step i-1 while step i runs, and for the last one at the end.
            # duplex: uploads and read-backs on two streams (both PCIe directions at once) or
            # on one (one direction at a time; faster where many GPUs share the host's links).
            main = torch.cuda.current_stream()
            back = back_stream if duplex else copy_stream
            with torch.cuda.stream(copy_stream):
                xin[0].copy_(hx, non_blocking=True)
                ready[0].record()
            for i in range(k):
                cur, nxt = i & 1, (i + 1) & 1
                if i + 1 < k:
                    with torch.cuda.stream(copy_stream):
                        if i >= 1:
                            copy_stream.wait_event(freed[nxt])
                        xin[nxt].copy_(hx, non_blocking=True)
                        ready[nxt].record()
                main.wait_event(ready[cur])
                if i >= 2:
                    main.wait_event(copied[cur])          # the output buffer has been read back
                comm.all_reduce(xin[cur], yout[cur], codec=args.codec, algo=args.algo, error_feedback=ef)
                freed[cur].record()
                done[cur].record()
                if full:
                    with torch.cuda.stream(back):
                        back.wait_event(done[cur])
                        hy[cur].copy_(yout[cur], non_blocking=True)
                        copied[cur].record()
                else:   # a metric of the result (its squared norm) instead of the result itself
                    metric = yout[cur].float().square().sum().reshape(1)
                    hm[cur].copy_(metric, non_blocking=True)
                    copied[cur].record()
                if i >= 1:
                    copied[nxt].synchronize()             # the host has step i-1's result
            copied[(k - 1) & 1].synchronize()
            main.wait_event(copied[(k - 1) & 1])

        def e2e_timed(k, duplex):
            barrier()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            e2e_loop(k, duplex)
            b.record()
            barrier()
            tt = torch.tensor([a.elapsed_time(b)], device=dev, dtype=torch.float64)
            if world > 1:
                dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            return tt.item() / k

        # which copy schedule this host prefers: measured on a few untimed steps, same on all ranks
        e2e_loop(2)
        trial = {True: e2e_timed(3, True), False: e2e_timed(3, False)}
        duplex = trial[True] <= trial[False]
        barrier()
        es, ee = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        es.record()
        t0 = time.perf_counter()
        e2e_loop(args.steps, duplex)
        ee.record()
        barrier()
        wall_ms = (time.perf_counter() - t0) * 1e3
        te = torch.tensor([max(es.elapsed_time(ee), 0.0)], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(te, op=dist.ReduceOp.MAX)
        e_ms = te.item() / args.steps
        # the same loop reading back a 4-byte metric of the result instead of the result: what
        # the upload and the collective cost without the second PCIe stream
        e2e_loop(2, duplex, False)
        metric_ms = 0.0
        barrier()
        ms0, ms1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ms0.record()
        e2e_loop(args.steps, duplex, False)
        ms1.record()
        barrier()
        tm = torch.tensor([ms0.elapsed_time(ms1)], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(tm, op=dist.ReduceOp.MAX)
        metric_ms = tm.item() / args.steps
        factor = 2 * (world - 1) / world if world > 1 else 1.0
        e2e = {"value": args.bytes / (e_ms * 1e-3) / 1e9 * factor * world, "unit": "GB/s",
               "busbw_per_gpu": args.bytes / (e_ms * 1e-3) / 1e9 * factor,
               "ms_per_step": e_ms, "wall_ms_per_step": wall_ms / args.steps,
               "h2d_bytes_per_step": args.bytes, "d2h_bytes_per_step": count * hy[0].element_size(),
               "metric_readback": {"ms_per_step": metric_ms, "d2h_bytes_per_step": 4,
                                   "value": args.bytes / (metric_ms * 1e-3) / 1e9 * factor * world,
                                   "note": "the same loop with the squared norm of the result read back instead of the result"},
               "copy_schedule": ("uploads and read-backs at once (two copy streams)" if duplex else
                                 "one PCIe direction at a time (one copy stream)"),
               "copy_schedule_trial_ms": {"both_directions_at_once": trial[True], "one_direction_at_a_time": trial[False]},
               "note": "pinned host input uploaded and the full result read back every step; the upload of step "
                       "i+1, the collective of step i and the read-back of step i-1 overlap (the host waits for "
                       "each step's result one step later); the copy schedule is the faster of two tried on "
                       "three untimed steps"}

    # ---- the same collective through the LD_PRELOAD interposer and the C benchmark driver ----
    interposed = None
    if args.via == "interposer" and world > 1:
        from ccbench_b200.bench import via_interposer

        interposed = via_interposer.run(x, rank=rank, world=world, local_rank=local_rank, nbytes=args.bytes, dtype=args.dtype,
                                        codec=args.codec, algo=args.algo, steps=args.steps, warmup=args.warmup)
        if rank == 0 and interposed and "ms_per_step" in interposed:
            interposed["direct_api_ms_per_step"] = ms_per_step
            interposed["interposed_over_direct"] = interposed["ms_per_step"] / ms_per_step

    factor = 2 * (world - 1) / world if world > 1 else 1.0
    algbw = args.bytes / (ms_per_step * 1e-3) / 1e9
    # roofline of the fused kernel: the wire bytes one GPU must push over NVLink at the
    # nominal 900 GB/s per direction (a copy-engine peer copy measures 770 GB/s, stores issued
    # by SMs 695 GB/s with traffic both ways: ccbench_b200.bench.linkprobe); one rank: input +
    # output at the measured 6553 GB/s copy bandwidth
    from ccbench_b200.comm import wire_bytes as _wire_bytes

    if world > 1:
        wire = factor * _wire_bytes(args.codec, dtype, count)
        bound_ms = wire / 900e9 * 1e3
        roofline = {"bound": "nvlink", "gbs": 900, "bound_ms": bound_ms, "fraction": bound_ms / ms_per_step,
                    "fraction_of_measured_770": wire / 770e9 * 1e3 / ms_per_step,
                    "fraction_of_sm_store_rate_695": wire / 695e9 * 1e3 / ms_per_step}
    else:
        bound_ms = 2 * args.bytes / 6553e9 * 1e3
        roofline = {"bound": "hbm", "gbs": 6553, "bound_ms": bound_ms, "fraction": bound_ms / ms_per_step}
    if rank == 0:
        line = {
            "metric": "compressed_allreduce_busbw",
            "value": algbw * factor * world, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "value_definition": "whole-job aggregate: per-GPU bus bandwidth (nccl-tests busbw = bytes/t * 2(n-1)/n; "
                                "algbw at n = 1) summed over the n GPUs; busbw_per_gpu holds the per-GPU figure",
            "busbw_per_gpu": algbw * factor,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": args.dtype, "data": "synthetic",
            "impl": "ours",
            "config": {"model": "gradient-like buffer: Laplace(0,1e-3) + 0.1% x100 outliers",
                       "global_batch": args.bytes * world, "seq_len": count,
                       "message_bytes_per_rank": args.bytes, "codec": args.codec, "algo": args.algo,
                       "algo_selection": ("measured before warm-up; ring (n requantisations) only if > 15 % faster than "
                                          "two-shot (2 requantisations)") if requested == "tune" else "fixed",
                       "algo_candidates": tuning, "pipelined_kernel": pipelined, "call_overlap": call_overlap,
                       "error_feedback": bool(args.error_feedback),
                       "parallelism": f"dp{world}", "l2": "inputs (256 MiB) larger than L2, no flush needed",
                       "busbw_formula": "bytes/t*2(n-1)/n; n=1 reports algbw"},
            "algbw": algbw, "ref_definition_bw": 2 * algbw, "compression_ratio": wire_ratio(args.codec, dtype),
            "rel_l2_error": rel_l2, "clocks": {k: clocks[k] for k in ("sm_mhz", "sm_max_mhz", "reasons")},
            "serialised_ms_per_step": serialised_ms, "e2e": e2e, "via_interposer": interposed, "gpu_launches": launches, "host_numa_binding": numa, "roofline": roofline,
        }
        print(json.dumps(line), flush=True)
    comm.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
