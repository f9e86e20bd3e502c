"""Parallelism strategies as communication workloads.

The reference implements none of DP / ZeRO / TP / SP / PP / EP / CP / Ulysses: it
benchmarks the collectives they emit, on tensors captured from a training run
(scripts/intermediate/generate_iter_datasets.py:32-81 names them: DP_AllGather weight
shards, DP_ReduceScatter grad shards, SP_ReduceScatter activations, PP_Comm send/recv,
...). Here each strategy is a first-class generator: from a model shape and a world
size it emits the exact list of collectives one training step issues (operation,
element count, dtype, repeat count, phase), and `run_plan` plays that list on a
Communicator with the fused compressed kernels, timing every entry on the device.

    python -m ccbench_b200.parallel.strategies --strategy zero3 --model llama-7b --world 8
    python -m torch.distributed.run --nproc-per-node 8 -m ccbench_b200.parallel.strategies \
        --strategy tp --model llama-7b --run --codec int8
"""
from __future__ import annotations

import argparse
import json
import math
import os
from dataclasses import asdict, dataclass


@dataclass(frozen=True)
class ModelShape:
    name: str
    layers: int
    hidden: int
    heads: int
    ffn: int
    vocab: int
    seq: int
    micro_batch: int = 1
    gated_mlp: bool = False      # Llama-style: three MLP matrices instead of two
    experts: int = 0             # > 0: every layer's MLP is a mixture of this many experts
    topk: int = 2

    @property
    def layer_params(self) -> int:
        attn = 4 * self.hidden * self.hidden
        mlp = (3 if self.gated_mlp else 2) * self.hidden * self.ffn
        if self.experts:
            mlp = mlp * self.experts + self.hidden * self.experts  # + router
        return attn + mlp + 4 * self.hidden  # + norms / biases, to first order

    @property
    def params(self) -> int:
        return self.layers * self.layer_params + self.vocab * self.hidden

    @property
    def tokens(self) -> int:
        return self.micro_batch * self.seq


PRESETS = {
    "gpt2-124m": ModelShape("gpt2-124m", 12, 768, 12, 3072, 50257, 1024, 8),
    "gpt2-1.5b": ModelShape("gpt2-1.5b", 48, 1600, 25, 6400, 50257, 1024, 4),
    "llama-7b": ModelShape("llama-7b", 32, 4096, 32, 11008, 32000, 4096, 1, gated_mlp=True),
    "llama-70b": ModelShape("llama-70b", 80, 8192, 64, 28672, 32000, 4096, 1, gated_mlp=True),
    "mixtral-8x7b": ModelShape("mixtral-8x7b", 32, 4096, 32, 14336, 32000, 4096, 1, gated_mlp=True, experts=8, topk=2),
}


@dataclass(frozen=True)
class CommOp:
    strategy: str
    phase: str          # fwd | bwd | opt
    collective: str     # allreduce | allgather | reducescatter | alltoall | sendrecv
    elems: int          # elements each rank contributes (allgather: its shard; others: the whole buffer)
    dtype: str
    repeat: int         # times per training step
    overlappable: bool  # can hide behind compute (bucketed gradients, prefetched weights)
    note: str = ""

    def bytes_per_rank(self) -> int:
        return self.elems * (4 if self.dtype == "f32" else 2)


def _buckets(total: int, bucket_elems: int):
    full, rest = divmod(total, bucket_elems)
    out = [(bucket_elems, full)] if full else []
    if rest:
        out.append((rest, 1))
    return out


def dp(m: ModelShape, world: int, bucket_mb: int = 25, dtype: str = "bf16"):
    """DDP: gradients all-reduced in buckets while backward still runs."""
    be = bucket_mb * (1 << 20) // (4 if dtype == "f32" else 2)
    return [CommOp("dp", "bwd", "allreduce", e, dtype, r, True, f"gradient bucket of {bucket_mb} MiB") for e, r in _buckets(m.params, be)]


def zero(m: ModelShape, world: int, stage: int = 3, bucket_mb: int = 25, dtype: str = "bf16"):
    """ZeRO / FSDP: stage 1-2 reduce-scatter gradients and all-gather updated weights once;
    stage 3 all-gathers every layer's weights in forward and again in backward."""
    be = bucket_mb * (1 << 20) // (4 if dtype == "f32" else 2)
    ops = [CommOp(f"zero{stage}", "bwd", "reducescatter", e, dtype, r, True, "gradient bucket -> owner shard")
           for e, r in _buckets(m.params, be)]
    if stage >= 3:
        shard = math.ceil(m.layer_params / world)
        ops.insert(0, CommOp("zero3", "fwd", "allgather", shard, dtype, m.layers, True, "layer weights before use"))
        ops.append(CommOp("zero3", "bwd", "allgather", shard, dtype, m.layers, True, "layer weights again for backward"))
        ops.append(CommOp("zero3", "fwd", "allgather", math.ceil(m.vocab * m.hidden / world), dtype, 2, True, "embedding / head"))
    else:
        ops.append(CommOp(f"zero{stage}", "opt", "allgather", math.ceil(m.params / world), dtype, 1, False, "updated weights"))
    return ops


def tp(m: ModelShape, world: int, dtype: str = "bf16"):
    """Megatron tensor parallel: one all-reduce after attention and one after the MLP, in
    forward and in backward, on [micro_batch, seq, hidden] activations (latency-critical)."""
    act = m.tokens * m.hidden
    return [CommOp("tp", ph, "allreduce", act, dtype, 2 * m.layers, False, "row-parallel output") for ph in ("fwd", "bwd")]


def sp(m: ModelShape, world: int, dtype: str = "bf16"):
    """Megatron sequence parallel: the TP all-reduce split into reduce-scatter + all-gather
    along the sequence, so norms and dropout run on a 1/world slice."""
    act = m.tokens * m.hidden
    ops = []
    for ph in ("fwd", "bwd"):
        ops.append(CommOp("sp", ph, "reducescatter", act, dtype, 2 * m.layers, False, "activations -> sequence shard"))
        ops.append(CommOp("sp", ph, "allgather", act // world, dtype, 2 * m.layers, False, "sequence shard -> activations"))
    return ops


def pp(m: ModelShape, world: int, microbatches: int = 8, dtype: str = "bf16"):
    """Pipeline parallel (1F1B): each stage boundary passes one activation forward and one
    gradient backward per micro-batch. Point-to-point; stays on NCCL send/recv."""
    act = m.tokens * m.hidden
    return [CommOp("pp", "fwd", "sendrecv", act, dtype, microbatches, True, "activation to the next stage"),
            CommOp("pp", "bwd", "sendrecv", act, dtype, microbatches, True, "gradient to the previous stage")]


def ep(m: ModelShape, world: int, dtype: str = "bf16"):
    """Expert parallel: per MoE layer a dispatch and a combine all-to-all of top-k routed
    token rows, forward and backward."""
    rows = m.tokens * m.topk * m.hidden
    return [CommOp("ep", ph, "alltoall", rows, dtype, 2 * m.layers, False, f"top-{m.topk} dispatch + combine") for ph in ("fwd", "bwd")]


def ulysses(m: ModelShape, world: int, dtype: str = "bf16"):
    """DeepSpeed-Ulysses: all-to-all that trades the sequence split for a head split on
    q, k, v before attention and on the output after it."""
    local = m.tokens // world * m.hidden
    return [CommOp("ulysses", ph, "alltoall", local, dtype, 4 * m.layers, False, "q, k, v, o: sequence <-> heads") for ph in ("fwd", "bwd")]


def cp(m: ModelShape, world: int, dtype: str = "bf16"):
    """Context parallel / ring attention: K and V blocks travel once around the ring per
    layer while the local attention block computes."""
    kv = 2 * (m.tokens // world) * m.hidden
    return [CommOp("cp", "fwd", "sendrecv", kv, dtype, (world - 1) * m.layers, True, "K,V block to the ring neighbour"),
            CommOp("cp", "bwd", "sendrecv", 2 * kv, dtype, (world - 1) * m.layers, True, "K,V and their gradients")]


STRATEGIES = {"dp": dp, "zero1": lambda m, w, **k: zero(m, w, stage=1, **k), "zero2": lambda m, w, **k: zero(m, w, stage=2, **k),
              "zero3": lambda m, w, **k: zero(m, w, stage=3, **k), "fsdp": lambda m, w, **k: zero(m, w, stage=3, **k),
              "tp": tp, "sp": sp, "pp": pp, "ep": ep, "ulysses": ulysses, "cp": cp}


def plan(strategy: str, model: str | ModelShape, world: int, **kw):
    m = PRESETS[model] if isinstance(model, str) else model
    return STRATEGIES[strategy](m, world, **kw)


def volume_bytes(ops, world: int) -> int:
    """Bytes each rank puts on the wire per step without compression (nccl-tests factors)."""
    tot = 0.0
    for o in ops:
        b = o.bytes_per_rank()
        f = {"allreduce": 2 * (world - 1) / world, "reducescatter": (world - 1) / world, "allgather": world - 1,
             "alltoall": (world - 1) / world, "sendrecv": 1.0}[o.collective]
        tot += b * f * o.repeat
    return int(tot)


def run_plan(comm, ops, *, codec: str = "int8", algo: str = "auto", move_codec: str | None = None, iters: int = 5,
             max_repeat: int = 4):
    """Plays the plan on `comm` (one process per GPU, or a local communicator with one
    tensor per emulated rank). Each entry is timed alone on the device (CUDA events,
    max over ranks when torch.distributed is up); `repeat` is capped at `max_repeat`
    launches per measurement and the total extrapolated. Send/recv entries use
    torch.distributed p2p between ring neighbours."""
    import torch
    import torch.distributed as dist

    from ..models.workloads import gradient_like, normal

    dev = torch.device("cuda", torch.cuda.current_device())
    n, nl = comm.nranks, comm.nlocal
    dist_up = dist.is_available() and dist.is_initialized()
    dts = {"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32}
    move = move_codec or ("fp8" if codec != "none" else "none")
    rows = []
    for o in ops:
        dt = dts[o.dtype]
        gen = gradient_like if o.phase != "fwd" or o.collective == "reducescatter" else normal
        elems = o.elems
        if o.collective in ("reducescatter", "alltoall"):
            elems = (elems + n - 1) // n * n
        send = [gen(elems, dt, seed=r, device=dev) for r in range(nl)]
        if o.collective == "allgather":
            recv = [torch.empty(elems * n, dtype=dt, device=dev) for _ in range(nl)]
        elif o.collective == "reducescatter":
            recv = [torch.empty(elems // n, dtype=dt, device=dev) for _ in range(nl)]
        else:
            recv = [torch.empty_like(s) for s in send]
        s_arg, r_arg = (send, recv) if nl > 1 else (send[0], recv[0])
        if o.collective == "allreduce":
            fn = lambda: comm.all_reduce(s_arg, r_arg, codec=codec, algo=algo)
        elif o.collective == "reducescatter":
            fn = lambda: comm.reduce_scatter(s_arg, r_arg, codec=codec)
        elif o.collective == "allgather":
            fn = lambda: comm.all_gather(s_arg, r_arg, codec=move)
        elif o.collective == "alltoall":
            fn = lambda: comm.all_to_all(s_arg, r_arg, codec=move)
        else:
            if not dist_up or dist.get_world_size() < 2:
                rows.append({**asdict(o), "time_us": None, "skipped": "send/recv needs torch.distributed with 2+ ranks"})
                continue
            rk, w = dist.get_rank(), dist.get_world_size()

            def fn():
                reqs = dist.batch_isend_irecv([dist.P2POp(dist.isend, send[0], (rk + 1) % w),
                                               dist.P2POp(dist.irecv, recv[0], (rk - 1) % w)])
                for q in reqs:
                    q.wait()
        reps = min(o.repeat, max_repeat)
        for _ in range(2):
            fn()
        if dist_up:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters * reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) * 1e3 / (iters * reps)], dtype=torch.float64, device=dev)
        if dist_up:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        us = t.item()
        rows.append({**asdict(o), "time_us": round(us, 2), "step_us": round(us * o.repeat, 1),
                     "algbw_GBs": round(o.bytes_per_rank() * (n if o.collective == "allgather" else 1) / us / 1e3, 2)})
        del send, recv
    return rows


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--strategy", required=True, choices=sorted(STRATEGIES))
    ap.add_argument("--model", default="llama-7b", choices=sorted(PRESETS))
    ap.add_argument("--world", type=int, default=int(os.environ.get("WORLD_SIZE", "8")))
    ap.add_argument("--run", action="store_true", help="play the plan on the GPUs (under torch.distributed.run for 2+ GPUs)")
    ap.add_argument("--codec", default="int8")
    ap.add_argument("--algo", default="auto")
    ap.add_argument("--iters", type=int, default=5)
    a = ap.parse_args(argv)
    ops = plan(a.strategy, a.model, a.world)
    if not a.run:
        for o in ops:
            print(json.dumps(asdict(o)))
        print(json.dumps({"strategy": a.strategy, "model": a.model, "world": a.world, "params": PRESETS[a.model].params,
                          "wire_bytes_per_rank_per_step_uncompressed": volume_bytes(ops, a.world)}))
        return 0
    import torch
    import torch.distributed as dist

    from .. import Communicator

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
        comm = Communicator.from_torch_distributed(arena_bytes=2 << 30)
    else:
        comm = Communicator.create(0, 1, f"strat{os.getpid()}", arena_bytes=2 << 30)
    ops = plan(a.strategy, a.model, world)
    for row in run_plan(comm, ops, codec=a.codec, algo=a.algo, iters=a.iters):
        if rank == 0:
            print(json.dumps(row), flush=True)
    comm.close()
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
