"""Glue between training loops and the fused compressed collectives.

* `CompressedAllReduceHook`: a `DistributedDataParallel.register_comm_hook` hook. Every
  gradient bucket is all-reduced by ONE fused kernel (codec + exchange + reduce) on the
  current stream, with an fp32 error-feedback residual kept per bucket, then averaged.
* `ShardedSync`: the ZeRO / FSDP pair on flat buffers: gradients are reduce-scattered to
  their owner shard (int8 by default), updated parameters all-gathered (fp8 by default).

Both only need an object with the `Communicator` methods they call, which is what the CPU
tests hand them. The reference has no training integration: it captures the collectives a
DDP run emits (`app_command ... --strategy dp`, userconfig/config_in_jsonc/
bench_basic_config.jsonc:59) and replays them.
"""
from __future__ import annotations

import torch


class CompressedAllReduceHook:
    """`ddp.register_comm_hook(state=None, hook=CompressedAllReduceHook(comm))`."""

    def __init__(self, comm, codec: str = "int8", algo: str = "auto", error_feedback: bool = True, min_numel: int = 0,
                 fallback=None):
        """min_numel: smaller buckets go to `fallback(tensor)` (for example torch.distributed's
        all_reduce) or, without one, through the communicator uncompressed."""
        self.comm, self.codec, self.algo = comm, codec, algo
        self.error_feedback, self.min_numel, self.fallback = error_feedback, min_numel, fallback
        self._residual: dict[tuple[int, int], torch.Tensor] = {}

    def residual(self, index: int, like: torch.Tensor) -> torch.Tensor | None:
        if not self.error_feedback:
            return None
        key = (index, like.numel())
        r = self._residual.get(key)
        if r is None or r.device != like.device:
            r = torch.zeros(like.numel(), dtype=torch.float32, device=like.device)
            self._residual[key] = r
        return r

    def state_dict(self) -> dict:
        return {f"{i}:{n}": r.detach().cpu() for (i, n), r in self._residual.items()}

    def load_state_dict(self, state: dict, device="cuda") -> None:
        self._residual = {tuple(int(x) for x in k.split(":")): v.to(device=device, dtype=torch.float32) for k, v in state.items()}

    def __call__(self, state, bucket):
        t = bucket.buffer()
        n = self.comm.nranks
        if t.numel() < self.min_numel:
            if self.fallback is not None:
                self.fallback(t)
            else:
                self.comm.all_reduce(t, codec="none", algo=self.algo)
        else:
            self.comm.all_reduce(t, codec=self.codec, algo=self.algo, error_feedback=self.residual(bucket.index(), t))
        t.div_(n)
        fut = torch.futures.Future()
        fut.set_result(t)   # the work is enqueued on the current stream, where DDP consumes it
        return fut


class ShardedSync:
    """Flat-buffer gradient / parameter synchronisation of sharded data parallelism.

    `grads` holds `nranks * shard` elements; after `reduce_gradients` this rank's `shard`
    holds the mean gradient of its slice. After the optimizer has updated the fp32 master
    slice, `gather_parameters` rebuilds the full low-precision parameter buffer everywhere."""

    def __init__(self, comm, grad_codec: str = "int8", param_codec: str = "fp8", error_feedback: bool = True):
        self.comm, self.grad_codec, self.param_codec = comm, grad_codec, param_codec
        self.error_feedback = error_feedback
        self._residual: torch.Tensor | None = None

    def reduce_gradients(self, grads: torch.Tensor, shard: torch.Tensor) -> torch.Tensor:
        n = self.comm.nranks
        if grads.numel() != shard.numel() * n:
            raise ValueError("grads must hold nranks * shard.numel() elements")
        ef = None
        if self.error_feedback:
            if self._residual is None or self._residual.numel() != grads.numel() or self._residual.device != grads.device:
                self._residual = torch.zeros(grads.numel(), dtype=torch.float32, device=grads.device)
            ef = self._residual
        self.comm.reduce_scatter(grads, shard, codec=self.grad_codec, error_feedback=ef)
        shard.div_(n)
        return shard

    def gather_parameters(self, shard: torch.Tensor, full: torch.Tensor) -> torch.Tensor:
        if full.numel() != shard.numel() * self.comm.nranks:
            raise ValueError("full must hold nranks * shard.numel() elements")
        self.comm.all_gather(shard, full, codec=self.param_codec)
        return full
