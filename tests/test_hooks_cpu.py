"""Training-loop glue against a stand-in communicator (plain torch on the CPU)."""
import torch

from ccbench_b200.parallel.hooks import CompressedAllReduceHook, ShardedSync


class FakeComm:
    """Pretends to be rank 0 of `n` ranks that all hold the same tensors."""

    def __init__(self, n):
        self.nranks, self.calls = n, []

    def all_reduce(self, t, recv=None, *, codec="int8", algo="auto", error_feedback=None):
        self.calls.append(("all_reduce", codec, t.numel(), error_feedback is not None))
        if error_feedback is not None:
            error_feedback += 1.0
        t.mul_(self.nranks)

    def reduce_scatter(self, send, recv, *, codec="int8", error_feedback=None):
        self.calls.append(("reduce_scatter", codec, send.numel(), error_feedback is not None))
        recv.copy_(send[: recv.numel()] * self.nranks)

    def all_gather(self, send, recv, *, codec="int8"):
        self.calls.append(("all_gather", codec, send.numel(), False))
        recv.copy_(send.repeat(self.nranks))


class Bucket:
    def __init__(self, idx, t):
        self._i, self._t = idx, t

    def index(self):
        return self._i

    def buffer(self):
        return self._t


def test_ddp_hook_averages_and_keeps_one_residual_per_bucket():
    comm = FakeComm(4)
    hook = CompressedAllReduceHook(comm, codec="fp8", min_numel=100)
    g0, g1, small = torch.ones(1000), torch.full((500,), 2.0), torch.ones(10)
    for _ in range(2):
        for i, g in enumerate((g0, g1, small)):
            out = hook(None, Bucket(i, g)).wait()
            assert out is g
    assert torch.allclose(g0, torch.ones(1000)) and torch.allclose(g1, torch.full((500,), 2.0))
    assert [c[1] for c in comm.calls[:3]] == ["fp8", "fp8", "none"] and comm.calls[2][3] is False
    st = hook.state_dict()
    assert set(st) == {"0:1000", "1:500"} and float(st["0:1000"][0]) == 2.0   # touched once per step
    other = CompressedAllReduceHook(comm)
    other.load_state_dict(st, device="cpu")
    assert torch.equal(other.residual(1, g1), st["1:500"])
    seen = []
    CompressedAllReduceHook(comm, min_numel=100, fallback=lambda t: seen.append(t.numel()))(None, Bucket(9, small))
    assert seen == [10]


def test_sharded_sync_shapes_and_means():
    comm = FakeComm(4)
    sync = ShardedSync(comm)
    grads, shard = torch.arange(40, dtype=torch.float32), torch.empty(10)
    sync.reduce_gradients(grads, shard)
    assert torch.allclose(shard, grads[:10]) and comm.calls[-1] == ("reduce_scatter", "int8", 40, True)
    full = torch.empty(40)
    sync.gather_parameters(shard, full)
    assert torch.equal(full, shard.repeat(4)) and comm.calls[-1][1] == "fp8"
    try:
        sync.reduce_gradients(grads, torch.empty(7))
    except ValueError:
        pass
    else:
        raise AssertionError("shape mismatch not refused")
