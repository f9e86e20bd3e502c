"""The work partition of the pipelined two-shot kernel, restated: every 512-element unit of
a shard belongs to exactly one (CTA, wave, item), waves are consecutive slices of a CTA's
chunks, and the table of wave boundaries that the kernel computes once per launch needs only
32-bit arithmetic (csrc/kernels/ccb_pipe.cuh: the `kb` table, `wave_items`, `item_elem`)."""
import random

import pytest

UNIT, CHUNK_UNITS = 512, 8


def wave_table(valid, b, G, W):
    units = (valid + UNIT - 1) // UNIT
    nch = (units + CHUNK_UNITS - 1) // CHUNK_UNITS
    K = (nch - b + G - 1) // G if nch > b else 0
    assert units < 2 ** 32 and K * W < 2 ** 64
    return [K * w // W for w in range(W + 1)]


def units_of(valid, b, G, W):
    kb = wave_table(valid, b, G, W)
    for w in range(W):
        items = (kb[w + 1] - kb[w]) * CHUNK_UNITS
        for i in range(items):
            ch = b + (kb[w] + (i >> 3)) * G
            unit = ch * CHUNK_UNITS + (i & 7)
            assert unit < 2 ** 32
            if unit * UNIT < valid:          # the kernel skips items past the end of the shard
                yield w, unit


@pytest.mark.parametrize("seed", range(6))
def test_every_unit_is_owned_once_and_waves_are_ordered(seed):
    rng = random.Random(seed)
    for _ in range(40):
        G = rng.choice([1, 2, 7, 37, 129, 148])
        W = rng.randint(1, 8)
        valid = rng.choice([1, 511, 512, 513, 4096, 4097, rng.randint(1, 3_000_000)])
        seen = {}
        for b in range(G):
            last_wave_of_chunk = {}
            for w, unit in units_of(valid, b, G, W):
                assert unit not in seen, (valid, G, W, unit)
                seen[unit] = (b, w)
                ch = unit // CHUNK_UNITS
                assert ch % G == b                                   # CTA b owns chunks b, b + G, ...
                assert last_wave_of_chunk.setdefault(ch, w) == w      # a chunk is never split between waves
        assert sorted(seen) == list(range((valid + UNIT - 1) // UNIT)), (valid, G, W)
        # the chunks of a CTA go to the waves in increasing order
        for b in range(G):
            order = [w for w, _ in units_of(valid, b, G, W)]
            assert order == sorted(order)


def test_empty_waves_and_empty_ctas_are_fine():
    assert list(units_of(100, 5, 8, 4)) == []                # one chunk in all, owned by CTA 0
    assert [u for _, u in units_of(100, 0, 8, 4)] == [0]
    assert wave_table(4096 * 3, 0, 1, 8) == [0, 0, 0, 1, 1, 1, 2, 2, 3]   # 3 chunks over 8 waves: some waves empty
