"""A model of the exchange pipeline's ordering rules (include/fwd_eb_shard.h, fwd_eb_pipeline_*),
run under random schedules on the CPU: with three buffer parts no rank ever writes into a part of a
peer's receive buffer that the peer has not folded yet, and no rank deadlocks; with two parts the
same rules do let such a write happen (so the model can tell the difference).

Rules modelled, per rank, for call e = 1, 2, ...:
  main stream   P(e): pool and write this rank's rows into part e % parts of every peer
                      — may start only after X(e-2) of the same rank has completed
  side stream   X(e): raise flag e on every peer; wait until every rank's flag >= e has arrived here;
                      fold part e % parts of the own buffer — starts after P(e) and after X(e-1)
Issuing the main stream's wait only on every k-th call (so that consecutive pooling grids are not
separated by a wait) needs k + 2 parts under these rules.

The fused-push steps of the pipeline as built go further: the flag of call e is raised by the
pooling grid itself when it completes (`flag_from_pool`), so the side stream's kernel only waits
and needs no hand-over from the main stream.  A flag then no longer proves that its rank has
folded the call before; the header's argument gives 2k + 2 parts as sufficient, and that variant
uses k = 3 with 8 parts.  The default (flag after the fold) uses k = 6 with the same 8 parts.
The schedule picks, at random, any operation whose predecessors have completed; operations of
different ranks and streams interleave freely.
"""
import random

import pytest


def simulate(world: int, parts: int, steps: int, seed: int, wait_every: int = 1,
             flag_from_pool: bool = False, depth: int = 2):
    rng = random.Random(seed)
    pooled = [0] * world          # last P completed per rank
    folded = [0] * world          # last X completed per rank (fold done)
    flags = [[0] * world for _ in range(world)]   # flags[owner][source]
    # what each part of each owner's buffer currently holds, per source: the call number written
    holds = [[[0] * world for _ in range(parts)] for _ in range(world)]
    hazards = []
    while min(folded) < steps:
        ready = []
        for r in range(world):
            e = pooled[r] + 1
            # the wait for X(e-2) is issued on every `wait_every`-th call only (1 = the pipeline as
            # built); the main stream being in order, later calls inherit the last wait
            waited_for = e - (e % wait_every) - depth
            if e <= steps and folded[r] >= waited_for:
                ready.append(("P", r, e))
            e = folded[r] + 1
            if e <= steps and (flag_from_pool or pooled[r] >= e):
                ready.append(("X", r, e))
        if not ready:
            return "deadlock", hazards
        kind, r, e = rng.choice(ready)
        if kind == "P":
            for owner in range(world):
                slot = holds[owner][e % parts]
                # the part must have been folded by its owner before it is overwritten
                if slot[r] != 0 and folded[owner] < slot[r]:
                    hazards.append((r, owner, e, slot[r], folded[owner]))
                slot[r] = e
            pooled[r] = e
            if flag_from_pool:
                for owner in range(world):
                    flags[owner][r] = max(flags[owner][r], e)
        else:
            if not flag_from_pool:
                for owner in range(world):
                    flags[owner][r] = max(flags[owner][r], e)
            if all(f >= e for f in flags[r]):
                # every source's rows of call e must be what the part holds now
                if any(holds[r][e % parts][src] != e for src in range(world)):
                    hazards.append(("stale", r, e, list(holds[r][e % parts])))
                folded[r] = e
            # else: the wait kernel keeps spinning; it is re-picked later (flags only grow)
    return "done", hazards


@pytest.mark.parametrize("world", [2, 3, 8])
def test_three_parts_never_overwrite_an_unfolded_part(world):
    for seed in range(200):
        state, hazards = simulate(world, parts=3, steps=12, seed=seed)
        assert state == "done" and not hazards, (seed, state, hazards[:3])


def test_two_parts_are_not_enough_under_the_same_rules():
    found = 0
    for seed in range(200):
        state, hazards = simulate(4, parts=2, steps=12, seed=seed)
        assert state == "done"
        found += bool(hazards)
    assert found > 0


@pytest.mark.parametrize("wait_every,parts,safe", [(2, 3, False), (2, 4, True), (3, 4, False), (3, 5, True)])
def test_waiting_on_every_kth_call_needs_k_plus_two_parts(wait_every, parts, safe):
    hazardous = 0
    for seed in range(200):
        state, hazards = simulate(4, parts=parts, steps=24, seed=seed, wait_every=wait_every)
        assert state == "done"
        hazardous += bool(hazards)
    assert (hazardous == 0) == safe


@pytest.mark.parametrize("world", [2, 4, 8])
def test_the_pipeline_as_built_wait_every_sixth_call_eight_parts(world):
    """The default: flag raised after the fold of the call before, a wait on every 6th call."""
    for seed in range(300):
        state, hazards = simulate(world, parts=8, steps=60, seed=seed, wait_every=6)
        assert state == "done" and not hazards, (seed, state, hazards[:3])
    bad = sum(bool(simulate(4, parts=7, steps=60, seed=seed, wait_every=6)[1]) for seed in range(300))
    assert bad > 0          # one part fewer does let a rank overwrite an unfolded part


@pytest.mark.parametrize("every,depth", [(8, 8), (4, 4), (12, 4), (2, 6)])
def test_lookback_every_k_calls_for_call_e_minus_d_needs_k_plus_d_parts(every, depth):
    """fwd_eb_pipeline_set_lookback: any (every, depth) is safe with every + depth parts."""
    for seed in range(150):
        state, hazards = simulate(4, parts=every + depth, steps=80, seed=seed, wait_every=every, depth=depth)
        assert state == "done" and not hazards, (seed, state, hazards[:3])
    bad = sum(bool(simulate(4, parts=every + depth - 1, steps=80, seed=seed, wait_every=every, depth=depth)[1])
              for seed in range(300))
    assert bad > 0


@pytest.mark.parametrize("world", [2, 4, 8])
def test_the_ticket_variant_flag_from_the_pooling_grid_wait_every_third_call_eight_parts(world):
    for seed in range(300):
        state, hazards = simulate(world, parts=8, steps=40, seed=seed, wait_every=3, flag_from_pool=True)
        assert state == "done" and not hazards, (seed, state, hazards[:3])


@pytest.mark.parametrize("wait_every,parts", [(1, 3), (2, 4), (3, 5)])
def test_flag_from_the_pooling_grid_needs_more_parts_than_flag_after_the_fold(wait_every, parts):
    """k + 2 parts, enough when a flag is raised only after the previous fold, are not enough once
    the pooling grid raises it."""
    hazardous = 0
    for seed in range(300):
        state, hazards = simulate(4, parts=parts, steps=30, seed=seed, wait_every=wait_every,
                                  flag_from_pool=True)
        assert state == "done"
        hazardous += bool(hazards)
    assert hazardous > 0


def simulate_lanes(world: int, parts: int, steps: int, seed: int, every: int, depth: int, lanes: int):
    """The same model with a rank's steps issued on `lanes` alternating caller streams (step e on
    stream e % lanes; a stream runs its steps in order, different streams run freely) and the
    look-back kept per stream as pipeline_begin keeps it: a step waits for this rank's fold of
    e - depth unless its stream is already behind a fold >= e - (every - 1) - depth."""
    rng = random.Random(seed)
    # the host decides the waits in issue order (the same on every rank)
    waited = [0] * lanes
    wait_for = [0] * (steps + 1)
    for e in range(1, steps + 1):
        lane = e % lanes
        if e > depth and waited[lane] + (every - 1) + depth < e:
            wait_for[e] = e - depth
            waited[lane] = e - depth
    done_p = [set() for _ in range(world)]
    lane_next = [[next((e for e in range(1, steps + 1) if e % lanes == lane), None) for lane in range(lanes)]
                 for _ in range(world)]
    folded = [0] * world
    flags = [[0] * world for _ in range(world)]
    holds = [[[0] * world for _ in range(parts)] for _ in range(world)]
    hazards = []
    while min(folded) < steps:
        ready = []
        for r in range(world):
            for lane in range(lanes):
                e = lane_next[r][lane]
                if e is not None and e <= steps and folded[r] >= wait_for[e]:
                    ready.append(("P", r, e, lane))
            e = folded[r] + 1
            if e <= steps and e in done_p[r]:
                ready.append(("X", r, e, 0))
        if not ready:
            return "deadlock", hazards
        kind, r, e, lane = rng.choice(ready)
        if kind == "P":
            for owner in range(world):
                slot = holds[owner][e % parts]
                if slot[r] != 0 and folded[owner] < slot[r]:
                    hazards.append((r, owner, e, slot[r], folded[owner]))
                slot[r] = e
            done_p[r].add(e)
            nxt = e + lanes
            lane_next[r][lane] = nxt if nxt <= steps else None
        else:
            for owner in range(world):
                flags[owner][r] = max(flags[owner][r], e)
            if all(f >= e for f in flags[r]):
                if any(holds[r][e % parts][src] != e for src in range(world)):
                    hazards.append(("stale", r, e, list(holds[r][e % parts])))
                folded[r] = e
    return "done", hazards


@pytest.mark.parametrize("lanes", [1, 2, 3])
@pytest.mark.parametrize("every,depth", [(6, 2), (8, 8), (1, 2), (4, 4)])
def test_steps_on_alternating_caller_streams_keep_the_k_plus_d_parts_rule(lanes, every, depth):
    for seed in range(60):
        state, hazards = simulate_lanes(4, every + depth, 60, seed, every, depth, lanes)
        assert state == "done" and not hazards, (seed, state, hazards[:3])
    if lanes == 1:          # on one stream the rule is tight: one part fewer is one too few
        bad = sum(bool(simulate_lanes(4, every + depth - 1, 60, seed, every, depth, lanes)[1]) for seed in range(200))
        assert bad > 0
