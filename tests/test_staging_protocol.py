"""The hand-off of the attention kernel's one output staging tile (csrc/sdpa_sm100.cu), modelled on the CPU.

Two query tiles take turns writing the staging tile; a store warp reads each use out (tile stores to every
destination) and signals "free".  A wait on an mbarrier sees only the PARITY of a phase, so a waiter must never be
two phases behind the barrier it waits on -- and here it can be: tile 1 comes to wait for use u + 1 while use u - 1
is still being read out and tile 0 has not staged use u yet; the barrier is then in phase u - 1, whose parity
equals that of phase u + 1, and the wait returns at once.  (This happened with eight destinations per tile.)  One
barrier per parity of the use number cures that case but not a tile that sat out an item or two.  The kernel
therefore signals "free" through a counter that only grows.  This model runs the three protocols under random
interleavings: both barrier protocols must be caught, the counter never.
"""
import random


class Barrier:
    """An mbarrier with one expected arrival per phase; waits test the parity of a phase for completion."""

    def __init__(self):
        self.phase = 0

    def arrive(self):
        self.phase += 1

    def done(self, parity):          # mbarrier.test_wait.parity: has the phase with this parity completed?
        return (self.phase & 1) != parity


def run(protocol, uses_of_tile, seed, steps=4000):
    """uses_of_tile[u] = which tile (0 / 1) stages use u.  Returns the first protocol violation or None."""
    rng = random.Random(seed)
    n = len(uses_of_tile)
    full = Barrier()
    free = [Barrier(), Barrier()]
    freed = 0                                 # the counter: uses read out so far
    next_use = {0: 0, 1: 0}                   # index into each tile's own list of uses
    mine = {t: [u for u in range(n) if uses_of_tile[u] == t] for t in (0, 1)}
    store_u, reading, owner = 0, False, None  # the store warp's use, whether it is reading the tile, who wrote it last
    staged = 0

    def tile_can_stage(t):
        if next_use[t] >= len(mine[t]):
            return False
        u = mine[t][next_use[t]]
        if protocol == "counter":
            return freed >= u
        if u == 0:
            return True
        if protocol == "barrier per parity":
            return free[(u - 1) & 1].done(((u - 1) >> 1) & 1)
        return free[0].done((u & 1) ^ 1)

    for _ in range(steps):
        actors = [("tile", t) for t in (0, 1) if tile_can_stage(t)]
        if not reading and store_u < n and full.done(store_u & 1):
            actors.append(("store begins", None))
        if reading:
            actors.append(("store ends", None))
        if not actors:
            break
        kind, t = rng.choice(actors)
        if kind == "tile":
            u = mine[t][next_use[t]]
            if reading:
                return f"use {u} written while use {store_u} is being read out"
            if u != staged:
                return f"use {u} staged out of turn (next is {staged})"
            staged += 1
            owner = u
            next_use[t] += 1
            full.arrive()
        elif kind == "store begins":
            if owner != store_u:
                return f"store warp reads use {store_u} but the tile holds use {owner}"
            reading = True
        else:
            reading = False
            free[store_u & 1 if protocol == "barrier per parity" else 0].arrive()
            freed += 1
            store_u += 1
    return None if staged == n and store_u == n else f"stuck after {staged} of {n} uses"


ALTERNATING = [u & 1 for u in range(24)]                         # both tiles have work in every item
IRREGULAR = [0, 1, 0, 1, 0, 0, 1, 0, 1, 1, 0, 0, 0, 1, 0, 1]     # items in which one tile has no rows
ONE_TILE = [0] * 12                                              # 256-wide heads, or Sq <= 128


def test_the_counter_never_lets_a_tile_in_early():
    for pat in (ALTERNATING, IRREGULAR, ONE_TILE):
        for seed in range(300):
            assert run("counter", pat, seed) is None, (pat, seed)


def test_a_single_barrier_is_caught_two_phases_behind():
    assert any(run("single barrier", ALTERNATING, seed) is not None for seed in range(300))


def test_a_barrier_per_parity_is_caught_when_a_tile_sits_out():
    assert all(run("barrier per parity", ALTERNATING, seed) is None for seed in range(300))
    assert any(run("barrier per parity", IRREGULAR, seed) is not None for seed in range(300))
