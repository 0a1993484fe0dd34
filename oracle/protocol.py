"""A CPU simulator of the barrier-free reduction protocol across ranks (test infrastructure only).

It models what dlmrt/ops/csrc/tp_comm.cu:1-22 describes and what this library's kernels do, at row granularity:
every rank owns receive slots `[buffers][world][R][n]` and one OUT buffer per call site, all resting at the arrival
sentinel (0xFFFF lanes); an invocation `e` on a rank

  1. pushes row s*R + r of its partial into rank s's slot [e % buffers][rank][r],
  2. re-arms the slot buffer peers will write next ((e + buffers - 1) % buffers) and the previous OUT of its chain,
  3. for each row it owns waits until all `world` slots hold data, sums them in rank order in FP32 and stores the row
     into OUT on every rank,
  4. waits until its own OUT copy is complete.

`one_shot=True` models the one-hop variant for small partials: slots are `[buffers][world][rows][n]`, every rank stores
its whole partial into every rank's slots and then sums ALL rows itself into its own OUT (no broadcast, no wait on OUT).

Ranks run as generators; a scheduler interleaves their steps in any order (seeded random, or a caller-supplied
priority), which is how the protocol's claim is tested: with three buffers no interleaving loses data, with two some
do. A rank that never pushes makes the others exhaust their wait budget: `ProtocolTimeout` names the waiting rank,
as the kernels' status words would (no GPU involved: failures are injected here on the host).
"""

import random

import numpy as np

from . import reduce as red
from .bf16 import SENTINEL, f32_to_bf16


class ProtocolTimeout(RuntimeError):
    def __init__(self, rank, what):
        super().__init__(f"rank {rank}: data never arrived ({what})")
        self.rank, self.what = rank, what


class Rank:
    def __init__(self, rank, world, rows, n, buffers, sites, one_shot=False):
        self.rank, self.world, self.R, self.n, self.buffers = rank, world, rows // world, n, buffers
        self.rows, self.one_shot = rows, one_shot
        self.recv = np.full((buffers, world, rows if one_shot else self.R, n), SENTINEL, dtype=np.uint16)
        self.out = {s: np.full((rows, n), SENTINEL, dtype=np.uint16) for s in sites}
        self.epoch = 0
        self.last_site = None
        self.results = []  # snapshot of OUT as the invocation's consumer would read it


def arrived(row):
    return not (row == SENTINEL).any()


def invocation(me, ranks, partial, site, late_rearm, silent=False):
    """Generator: one reduction on rank `me`. Yields True after a step that made progress, False when blocked."""
    world, R = me.world, me.R
    e = me.epoch + 1
    buf = e % me.buffers
    if not silent:  # a silent rank runs the kernel but its pushes go nowhere (fault injection)
        if me.one_shot:
            for row in range(me.rows):  # the whole partial, to every rank (peers first, as the stores rotate)
                for d in range(world):
                    ranks[(me.rank + d) % world].recv[buf, me.rank, row] = partial[row]
                    yield True
        else:
            for l in range(world * R):  # destinations rotate so that first stores spread over the peers
                r, s = l // world, (me.rank + l % world) % world
                ranks[s].recv[buf, me.rank, r] = partial[s * R + r]
                yield True

    def rearm():
        me.recv[(e + me.buffers - 1) % me.buffers] = SENTINEL
        if me.last_site is not None:
            me.out[me.last_site][:] = SENTINEL

    if not late_rearm:
        rearm()
        yield True
    for r in range(me.rows if me.one_shot else R):
        while not all(arrived(me.recv[buf, s, r]) for s in range(world)):
            yield False
        row = f32_to_bf16(red.rank_order_sum(me.recv[buf, :, r][:, None, :]))[0]  # rank order, FP32, from +0.0f
        if me.one_shot:
            me.out[site][r] = row  # every rank computes every row: nothing to broadcast
        else:
            for peer in ranks:
                peer.out[site][me.rank * R + r] = row
        yield True
    while not me.one_shot and not all(arrived(me.out[site][j]) for j in range(world * R)):
        yield False
    me.results.append(me.out[site].copy())
    if late_rearm:
        rearm()
        yield True
    me.epoch = e
    me.last_site = site


def run(world, rows, n, calls, buffers=3, seed=0, late_rearm=False, priority=None, silent_rank=None, budget=20000,
        one_shot=False):
    """Runs `calls` = [(site, partials [world, rows, n])] on all ranks under a random (or prioritised) interleaving.
    Returns each rank's list of OUT snapshots. Raises ProtocolTimeout when ranks stay blocked for `budget` picks."""
    sites = sorted({s for s, _ in calls})
    ranks = [Rank(r, world, rows, n, buffers, sites, one_shot) for r in range(world)]
    rng = random.Random(seed)
    todo = [list(calls) for _ in range(world)]
    running = [None] * world
    idle = 0
    blocked = set()  # ranks whose last step found nothing to do; cleared whenever any rank makes progress
    while any(todo) or any(g is not None for g in running):
        alive = [r for r in range(world) if running[r] is not None or todo[r]]
        r = priority(alive, blocked, rng) if priority else rng.choice(alive)
        if running[r] is None:
            site, partials = todo[r].pop(0)
            running[r] = invocation(ranks[r], ranks, partials[r], site, late_rearm, silent=(r == silent_rank))
        try:
            progressed = next(running[r])
        except StopIteration:
            running[r], progressed = None, True
        idle = 0 if progressed else idle + 1
        if progressed:
            blocked.clear()
        else:
            blocked.add(r)
        if idle > budget:
            raise ProtocolTimeout(r, "receive slots or OUT rows still hold the sentinel")
    return [rk.results for rk in ranks]
