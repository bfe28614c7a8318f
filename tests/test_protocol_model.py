"""CPU models of the flag protocols of the peer-memory kernels, run under random interleavings of the ranks.

Each rank is a generator that yields after every globally visible memory operation; a scheduler picks which rank
moves next.  The models state the protocol of ``csrc/comm_allreduce.cu`` (epoch flags + receive buffers alternating
by call parity; value-is-the-flag slots rotating over three arrays) and check the invariant the kernels rely on:
a reader only ever sees the values of ITS call.  The same models with one buffer fewer must break under some
schedule - which shows the checks can fail.
"""
import random

import pytest


def run(ranks, seed, max_steps=200_000):
    rng = random.Random(seed)
    live = list(ranks)
    steps = 0
    while live:
        g = rng.choice(live)
        try:
            next(g)
        except StopIteration:
            live.remove(g)
        steps += 1
        assert steps < max_steps, "protocol model did not terminate (deadlock)"


class Stale(Exception):
    pass


# ------------------------------------------------------------------------------------------- one-shot all-reduce
def allreduce_rank(r, n, calls, mem, buffers):
    """Push my value of call c into every rank's slot [c % buffers][r], raise my flag to c, wait for all flags,
    read all slots of my own buffer."""
    for c in range(1, calls + 1):
        p = c % buffers
        for d in range(n):
            mem["recv"][d][p][r] = (c, r)
            yield
        for d in range(n):
            mem["flag"][d][r] = c                       # release: ordered after the stores above
            yield
        for s in range(n):
            while mem["flag"][r][s] < c:                # acquire
                yield
        for s in range(n):
            if mem["recv"][r][p][s] != (c, s):
                raise Stale(f"rank {r} call {c}: slot of {s} holds {mem['recv'][r][p][s]}")
            yield


def allreduce_world(n, buffers):
    return {"recv": [[[None] * n for _ in range(buffers)] for _ in range(n)], "flag": [[0] * n for _ in range(n)]}


@pytest.mark.parametrize("n", [2, 4, 8])
def test_allreduce_parity_buffers_are_enough(n):
    for seed in range(60):
        mem = allreduce_world(n, 2)
        run([allreduce_rank(r, n, 6, mem, 2) for r in range(n)], seed)


def test_allreduce_single_buffer_is_not_enough():
    broken = 0
    for seed in range(200):
        mem = allreduce_world(2, 1)
        try:
            run([allreduce_rank(r, 2, 6, mem, 1) for r in range(2)], seed)
        except Stale:
            broken += 1
    assert broken > 0


# ------------------------------------------------------------------------------------------- value-is-the-flag slots
EMPTY = "empty"


def rms_rank(r, n, calls, slots, arrays):
    """Call c uses array c % arrays: write my partial into every rank's slot [r], spin on my own slots until none
    is empty, then clear the array the PREVIOUS call used (its values have all been read)."""
    for c in range(calls):
        a, clear = c % arrays, (c - 1) % arrays
        for d in range(n):
            slots[d][a][r] = (c, r)
            yield
        for s in range(n):
            while slots[r][a][s] == EMPTY:
                yield
            if slots[r][a][s] != (c, s):
                raise Stale(f"rank {r} call {c}: slot of {s} holds {slots[r][a][s]}")
        if c > 0:
            for s in range(n):
                slots[r][clear][s] = EMPTY
                yield


def rms_world(n, arrays):
    return [[[EMPTY] * n for _ in range(arrays)] for _ in range(n)]


@pytest.mark.parametrize("n", [2, 4, 8])
def test_three_slot_arrays_are_enough(n):
    for seed in range(60):
        slots = rms_world(n, 3)
        run([rms_rank(r, n, 7, slots, 3) for r in range(n)], seed)


def test_two_slot_arrays_are_not_enough():
    """With two arrays a fast peer's write for call c + 1 can land in the array this rank is about to clear."""
    broken = 0
    for seed in range(300):
        slots = rms_world(2, 2)
        try:
            run([rms_rank(r, 2, 7, slots, 2) for r in range(2)], seed, max_steps=20_000)
        except (Stale, AssertionError):
            broken += 1
    assert broken > 0
