"""A model of the epoch-flag protocol the fused collectives use, run under random interleavings.

Every rank is a coroutine that yields before each access to memory other ranks can see; a scheduler picks the next
rank at random, so one run is one interleaving of the ranks' loads and stores.  Checked properties:

* barrier safety: nobody leaves the barrier of epoch ``e`` before everybody has announced ``e``;
* epochs are monotonic counters, so a flag left over from epoch ``e`` never satisfies a wait for ``e + 1`` and the
  flag array needs no reset between calls;
* the tensor-parallel all-gather keeps ONE barrier per call because it alternates two activation buffers: a shard
  is overwritten two calls later, after a barrier every reader has passed.  The same program with a single buffer
  is wrong, and the model finds the interleaving that shows it;
* a rank that never arrives makes the others give up after their bounded wait with a record of who was missing.
"""
import random

import pytest


class World:
    def __init__(self, world, buffers):
        self.world = world
        self.flags = [[0] * world for _ in range(world)]              # flags[owner][slot]
        self.act = [[None] * world for _ in range(buffers)]           # act[buffer][owner] = (call, owner)
        self.buffers = buffers
        self.left_barrier = [0] * world                               # last epoch each rank passed
        self.announced = [0] * world
        self.errors = []
        self.timeouts = []


def rank_program(w: World, r: int, calls: int, wait_limit: int = 10_000, absent: bool = False):
    """One rank of ``calls`` all-gather + consume rounds.  Yields before every shared-memory access."""
    if absent:
        return
    for c in range(calls):
        b = c % w.buffers
        yield
        w.act[b][r] = (c, r)                                          # publish this call's shard
        epoch = c + 1
        w.announced[r] = epoch                                        # arrived: its shard is published
        for p in range(w.world):                                      # announce (release stores to every peer)
            yield
            w.flags[p][r] = epoch
        for q in range(w.world):                                      # wait (acquire loads of the local array)
            polls = 0
            while True:
                yield
                if w.flags[r][q] >= epoch:
                    break
                polls += 1
                if polls > wait_limit:
                    w.timeouts.append({"rank": r, "peer": q, "expected": epoch, "seen": w.flags[r][q]})
                    return
        if min(w.announced) < epoch:
            w.errors.append(f"rank {r} left barrier {epoch} before everybody announced it")
        w.left_barrier[r] = epoch
        for q in range(w.world):                                      # the consumer reads every peer's shard
            yield
            if w.act[b][q] != (c, q):
                w.errors.append(f"rank {r}, call {c}: read {w.act[b][q]} from rank {q}")


def run(world, buffers, calls, seed, absent=(), wait_limit=10_000, bias=None):
    rng = random.Random(seed)
    w = World(world, buffers)
    live = {r: rank_program(w, r, calls, wait_limit, r in absent) for r in range(world)}
    steps = 0
    while live and steps < 2_000_000:
        ranks = sorted(live)
        weights = [(bias or {}).get(r, 1.0) for r in ranks]
        r = rng.choices(ranks, weights)[0]
        try:
            next(live[r])
        except StopIteration:
            del live[r]
        steps += 1
    assert not live, "the model did not terminate"
    return w


@pytest.mark.parametrize("world", [2, 3, 4])
def test_double_buffered_all_gather_is_safe_under_random_interleavings(world):
    for seed in range(60):
        # unequal speeds make a rank run far ahead of the others, which is where reuse bugs hide
        bias = {r: random.Random(seed * 31 + r).choice([0.05, 1.0, 20.0]) for r in range(world)}
        w = run(world, buffers=2, calls=6, seed=seed, bias=bias)
        assert w.errors == [] and w.timeouts == []
        assert w.left_barrier == [6] * world
        assert all(f == [6] * world for f in w.flags)                 # counters only ever grow: no reset needed


def test_single_buffer_with_one_barrier_is_caught():
    """With one buffer a fast rank overwrites its shard for call c + 1 while a slow rank still reads call c."""
    found = 0
    for seed in range(200):
        bias = {0: 20.0, 1: 0.05}
        w = run(2, buffers=1, calls=4, seed=seed, bias=bias)
        assert w.timeouts == []
        found += bool(w.errors)
    assert found > 0


def test_stale_epoch_does_not_satisfy_the_next_wait():
    """After three completed calls every slot holds 3.  A rank that starts call 4 alone must not get through on
    those left-over flags: the comparison is ``flag >= epoch`` against a counter that only grows."""
    w = World(2, 2)
    w.flags = [[3, 3], [3, 3]]
    w.announced = [3, 3]

    def fourth_call(r, limit=50):
        epoch = 4
        w.announced[r] = epoch
        for p in range(w.world):
            yield
            w.flags[p][r] = epoch
        for q in range(w.world):
            polls = 0
            while w.flags[r][q] < epoch:
                yield
                polls += 1
                if polls > limit:
                    w.timeouts.append({"rank": r, "peer": q, "expected": epoch, "seen": w.flags[r][q]})
                    return
        w.left_barrier[r] = epoch

    list(fourth_call(0))
    assert w.timeouts == [{"rank": 0, "peer": 1, "expected": 4, "seen": 3}] and w.left_barrier[0] == 0
    w.timeouts.clear()
    list(fourth_call(1))                                              # the peer arrives: both slots hold 4 now
    list(fourth_call(0))
    assert w.timeouts == [] and w.left_barrier == [4, 4]


@pytest.mark.parametrize("world,missing", [(2, 1), (4, 2)])
def test_absent_rank_ends_in_bounded_timeouts_with_a_record(world, missing):
    w = run(world, buffers=2, calls=3, seed=7, absent=(missing,), wait_limit=200)
    assert w.errors == []
    assert sorted(t["rank"] for t in w.timeouts) == [r for r in range(world) if r != missing]
    assert all(t["peer"] == missing and t["expected"] == 1 and t["seen"] == 0 for t in w.timeouts)
    assert all(w.left_barrier[r] == 0 for r in range(world))          # nobody consumed a shard that never came
