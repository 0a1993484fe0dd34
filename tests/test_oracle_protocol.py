"""The push / poll / re-arm protocol on the CPU simulator (oracle.protocol): no interleaving of the ranks loses data
with three receive buffers, some do with two, and a rank that never pushes is reported, not waited for forever."""

import numpy as np
import pytest

from oracle import protocol
from oracle import reduce as red
from oracle.bf16 import f32_to_bf16


def calls(world, rows, n, count, seed):
    rng = np.random.default_rng(seed)
    out = []
    for i in range(count):
        partials = f32_to_bf16(rng.standard_normal((world, rows, n)).astype(np.float32))
        out.append((f"site{i % 2}", partials))
    return out


@pytest.mark.parametrize("world", [1, 2, 4, 8])
@pytest.mark.parametrize("late_rearm", [False, True])
@pytest.mark.parametrize("one_shot", [False, True])
def test_every_interleaving_gives_the_oracle_result(world, late_rearm, one_shot):
    rows, n = 2 * world, 256
    work = calls(world, rows, n, 7, seed=world)
    for seed in range(6):
        results = protocol.run(world, rows, n, work, seed=seed, late_rearm=late_rearm, one_shot=one_shot)
        for i, (_, partials) in enumerate(work):
            want = red.reduce(partials)
            for r in range(world):
                assert np.array_equal(results[r][i], want), f"seed {seed} call {i} rank {r}"


def hurry(rank):
    """A scheduler that runs `rank` whenever it is not blocked, and the others only to unblock it."""
    def pick(alive, blocked, rng):
        if rank in alive and rank not in blocked:
            return rank
        others = [r for r in alive if r != rank and r not in blocked] or [r for r in alive if r != rank] or alive
        return rng.choice(others)
    return pick


def test_two_buffers_lose_data_three_do_not():
    """The reason for triple buffering (tp_comm.cu:16-22): with two buffers a rank that re-arms late wipes the pushes a
    faster peer already made for the next invocation."""
    world, rows, n = 2, 4, 256
    work = calls(world, rows, n, 6, seed=9)
    ok = protocol.run(world, rows, n, work, buffers=3, late_rearm=True, priority=hurry(1))
    for i, (_, partials) in enumerate(work):
        assert np.array_equal(ok[0][i], red.reduce(partials))
    failures = 0
    for seed in range(8):
        try:
            got = protocol.run(world, rows, n, work, buffers=2, late_rearm=True, priority=hurry(1), seed=seed, budget=2000)
            failures += any(not np.array_equal(got[r][i], red.reduce(p)) for r in range(world) for i, (_, p) in enumerate(work))
        except protocol.ProtocolTimeout:
            failures += 1
    assert failures > 0


def test_one_hop_variant_survives_a_hurried_rank_with_three_buffers():
    """One hop has no wait on OUT, so a fast rank runs further ahead of a slow one than in the two-hop protocol; three
    buffers still suffice because finishing invocation e needs every peer's push of e, made after that peer's e - 1."""
    world, rows, n = 4, 4, 256
    work = calls(world, rows, n, 9, seed=3)
    for fast in range(world):
        for late in (False, True):
            got = protocol.run(world, rows, n, work, late_rearm=late, priority=hurry(fast), one_shot=True)
            for i, (_, partials) in enumerate(work):
                for r in range(world):
                    assert np.array_equal(got[r][i], red.reduce(partials)), (fast, late, i, r)


def test_a_rank_that_never_pushes_is_reported():
    world, rows, n = 4, 8, 256
    with pytest.raises(protocol.ProtocolTimeout) as e:
        protocol.run(world, rows, n, calls(world, rows, n, 2, seed=1), silent_rank=2, budget=500)
    assert e.value.rank != -1 and "never arrived" in str(e.value)
