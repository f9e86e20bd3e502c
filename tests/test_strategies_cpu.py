"""Parallelism-strategy workload generators: volumes and shapes, no GPU."""
import math

import pytest

from ccbench_b200.parallel import strategies as S


@pytest.mark.parametrize("model", sorted(S.PRESETS))
def test_dp_covers_every_parameter(model):
    m = S.PRESETS[model]
    ops = S.plan("dp", model, 8)
    assert sum(o.elems * o.repeat for o in ops) == m.params
    assert all(o.collective == "allreduce" and o.overlappable for o in ops)
    assert max(o.bytes_per_rank() for o in ops) <= 25 << 20


def test_zero3_gathers_weights_twice_and_scatters_gradients_once():
    m, w = S.PRESETS["llama-7b"], 8
    ops = S.plan("zero3", "llama-7b", w)
    rs = sum(o.elems * o.repeat for o in ops if o.collective == "reducescatter")
    ag = sum(o.elems * o.repeat * w for o in ops if o.collective == "allgather")
    assert rs == m.params
    assert abs(ag - 2 * m.params) / m.params < 0.01
    z1 = S.plan("zero1", "llama-7b", w)
    assert [o.collective for o in z1 if o.phase == "opt"] == ["allgather"]


def test_tp_sp_volumes_agree():
    w = 8
    tp, sp = S.plan("tp", "llama-7b", w), S.plan("sp", "llama-7b", w)
    # reduce-scatter + all-gather moves exactly what the all-reduce it replaces moves
    assert S.volume_bytes(tp, w) == S.volume_bytes(sp, w)
    assert sum(o.repeat for o in tp) == 4 * S.PRESETS["llama-7b"].layers


def test_point_to_point_and_all_to_all_strategies():
    m, w = S.PRESETS["mixtral-8x7b"], 8
    ep = S.plan("ep", "mixtral-8x7b", w)
    assert all(o.collective == "alltoall" and o.elems == m.tokens * m.topk * m.hidden for o in ep)
    assert {o.collective for o in S.plan("pp", "gpt2-1.5b", 4)} == {"sendrecv"}
    cp = S.plan("cp", "llama-7b", w)
    assert cp[0].repeat == (w - 1) * S.PRESETS["llama-7b"].layers
    ul = S.plan("ulysses", "llama-7b", w)
    assert ul[0].elems == S.PRESETS["llama-7b"].tokens // w * 4096


def test_cli_prints_the_plan(capsys):
    assert S.main(["--strategy", "zero3", "--model", "gpt2-124m", "--world", "4"]) == 0
    out = capsys.readouterr().out.strip().splitlines()
    assert "wire_bytes_per_rank_per_step_uncompressed" in out[-1]
    assert math.isfinite(float(len(out)))
