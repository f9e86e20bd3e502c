"""The mailbox protocol of the point-to-point kernel as a state machine, run under random
interleavings of the two ends (csrc/kernels/ccb_p2p.cuh): two halves per (source, lane), a
counter of rounds delivered in the receiver's arena and a counter of rounds consumed in the
sender's. Checked: every round is read exactly once and before its half is written again,
across several messages whose round numbers keep counting, and neither end can block for
ever when the other keeps running."""
import random

import pytest


class Lane:
    def __init__(self):
        self.box = [None, None]   # what the two halves hold: (round, payload)
        self.data = 0             # rounds delivered (written by the sender, in the receiver's arena)
        self.ack = 0              # rounds consumed (written by the receiver, in the sender's arena)


def sender(lane, first_round, rounds, payload):
    """Generator: one yield per step that touches shared state."""
    for k in range(rounds):
        g = first_round + k
        while not (g < 2 or lane.ack >= g - 1):     # the half is free once round g - 2 was consumed
            yield "wait"
        lane.box[g & 1] = (g, payload(g))
        yield "stored"
        lane.data = g + 1                            # published after the stores (release)
        yield "signalled"


def receiver(lane, first_round, rounds, out):
    for k in range(rounds):
        g = first_round + k
        while lane.data < g + 1:
            yield "wait"
        tag, value = lane.box[g & 1]
        assert tag == g, f"round {g} read a half that holds round {tag}"
        out.append(value)
        yield "copied"
        lane.ack = g + 1                             # only after every thread has read the half
        yield "acked"


@pytest.mark.parametrize("seed", range(8))
def test_rounds_arrive_once_in_order_under_any_interleaving(seed):
    rng = random.Random(seed)
    lane = Lane()
    sent = recvd = 0
    got = []
    messages = [rng.randint(1, 7) for _ in range(12)]       # rounds per message; counters never reset
    for rounds in messages:
        s = sender(lane, sent, rounds, lambda g: g * 10 + 1)
        r = receiver(lane, recvd, rounds, got)
        alive = {"s": s, "r": r}
        idle = 0
        while alive:
            who = rng.choice(sorted(alive))
            # bias: sometimes let one end run far ahead of the other
            for _ in range(rng.choice([1, 1, 1, 5, 20])):
                try:
                    step = next(alive[who])
                except StopIteration:
                    del alive[who]
                    break
                idle = idle + 1 if step == "wait" else 0
                assert idle < 10_000, "both ends wait: deadlock"
                if step == "wait":
                    break
        sent += rounds
        recvd += rounds
    assert got == [g * 10 + 1 for g in range(sum(messages))]


def test_a_sender_runs_at_most_two_rounds_ahead():
    lane = Lane()
    s = sender(lane, 0, 5, lambda g: g)
    steps = []
    for _ in range(50):
        steps.append(next(s))
        if steps[-1] == "wait" and steps.count("wait") > 5:
            break
    assert lane.data == 2 and steps.count("signalled") == 2    # two halves filled, then it waits for an acknowledgement
