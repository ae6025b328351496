"""Model check of the exchange protocol of csrc/gn_peer.cuh (CPU, no CUDA).

The device code cannot run without one GPU per rank, so its protocol - push numbers, the two slot
parities, the acknowledgement that travels with the next push, the wait before a slot is reused - is
restated here step by step in Python and run under many random interleavings of the ranks.  Checked:
  * safety: a slot is never overwritten before its owner has finished reading the values of the push
    before last (the property the acknowledgements exist for);
  * every collect returns the sum of that push's values over all ranks, identically on every rank;
  * liveness: every legal call sequence (at most two pushes outstanding) finishes, in particular the
    sequence where every rank is about to wait for exactly the acknowledgement it has not sent yet;
  * an illegal sequence (a third push before the first collect) cannot finish: the model reports the
    wait that the kernels would bound and count.
Each `yield` is one memory access of the device code, so the scheduler can switch ranks between any two.
"""
import random

import pytest


class Rank:
    def __init__(self, world):
        # the rank's exchange buffer, written by every rank
        self.slot = [[(0.0, 0) for _ in range(world)] for _ in range(2)]  # [parity][source rank] = (value, number)
        self.ack = [0] * world  # [rank q] = last collect q has acknowledged
        # words only the owner touches
        self.pushed = self.collected = self.done = self.acked = 0


def push(ranks, r, value, log):
    me, world = ranks[r], len(ranks)
    seq, fin, old = me.pushed + 1, me.done, me.acked
    me.pushed, me.acked = seq, fin
    if fin != old:  # first of all: which slots this rank has finished reading
        for q in range(world):
            yield "step"
            ranks[q].ack[r] = fin
    if seq > 2:  # the slots of push seq - 2 are free once every rank has collected it
        for q in range(world):
            while me.ack[q] < seq - 2:
                yield "wait"
    for q in range(world):
        yield "step"
        # safety: rank q must have finished reading what this store overwrites
        assert ranks[q].done >= seq - 2, "rank %d overwrites push %d in rank %d's buffer, which has read up to %d" % (
            r, seq - 2, q, ranks[q].done)
        ranks[q].slot[seq & 1][r] = (value, seq)
    log.append(("push", r, seq))


def collect(ranks, r, out):
    me, world = ranks[r], len(ranks)
    seq = me.collected + 1
    me.collected = seq
    total = 0.0
    for q in range(world):  # rank order
        while True:
            yield "wait" if me.slot[seq & 1][q][1] != seq else "step"
            value, number = me.slot[seq & 1][q]
            if number == seq:
                break
        total += value
    me.done = seq
    out.append((seq, total))


def program(ranks, r, calls, out, log):
    """calls: string of 'P' (push), 'C' (collect), 'A' (push + collect in one kernel)."""
    n = 0
    for op in calls:
        if op in "PA":
            n += 1
            yield from push(ranks, r, float((r + 1) * 100 + n), log)
        if op in "CA":
            yield from collect(ranks, r, out)


def run(world, calls, seed, max_idle=20000):
    rng = random.Random(seed)
    ranks = [Rank(world) for _ in range(world)]
    outs, log = [[] for _ in range(world)], []
    gens = {r: program(ranks, r, calls, outs[r], log) for r in range(world)}
    idle = 0
    while gens:
        r = rng.choice(list(gens))
        try:
            state = next(gens[r])
        except StopIteration:
            del gens[r]
            idle = 0
            continue
        idle = idle + 1 if state == "wait" else 0
        if idle > max_idle:  # every scheduled rank has only been waiting: the kernels would give up here
            return None
    return outs


LEGAL = ["AAAAAA", "PCPCPCPC", "PPCCPPCCPPCC", "PPCPCPCC", "APPCCAPCA", "PPCCAAPPCC"]


@pytest.mark.parametrize("world", [2, 3, 8])
@pytest.mark.parametrize("calls", LEGAL)
def test_legal_sequences_finish_with_the_right_sums(world, calls):
    for seed in range(40):
        outs = run(world, calls, seed)
        assert outs is not None, "deadlock in %s at seed %d" % (calls, seed)
        pushes = sum(op in "PA" for op in calls)
        want = [(n, float(sum((q + 1) * 100 + n for q in range(world)))) for n in range(1, pushes + 1)]
        for r in range(world):
            assert outs[r] == want, (calls, seed, r)


def test_every_rank_waiting_for_the_acknowledgement_it_owes_does_not_deadlock():
    # push 3 of every rank needs all acknowledgements of collect 1, which travel with ... push 3: each
    # rank must send its own before it waits for the others'
    for seed in range(200):
        assert run(4, "PPCCP", seed) is not None


def test_a_third_outstanding_push_cannot_finish():
    # no rank has collected push 1, so nobody ever acknowledges it: the model sees the wait that the
    # kernels bound (and report through gnb200_wait_timeouts)
    assert run(2, "PPPCCC", 0, max_idle=2000) is None
