"""The flag protocol of the o_proj exchange (pie_b200/csrc/oproj_reduce.cu), replayed on the CPU.

Kernels that wait for one another cannot be emulated as separate launches on one GPU, so the order in which
the ranks' CTAs may interleave is explored here instead: a model of the epilogue's state machine (senders
store a partial and raise a flag; owners wait for every sender of the tile, read the staged partials, store
the result rows into every rank's buffer and raise the completion flags; a CTA waits for the completion
flags of its tiles before it retires; a rank's next launch starts when its previous one has retired and its
consumer has read the result) is run under seeded random schedules.  Checked: every schedule finishes (no
cycle of waits), an owner only ever reads partials of its own tile and step (the staging is never
overwritten early nor read late), and a rank's consumer always finds the rows of the step it waits for (two
alternating output buffers are enough although ranks run ahead of one another)."""
import random

import pytest


def run_schedule(world, grid, tiles, steps, seed):
    rng = random.Random(seed)
    slots = -(-tiles // world)
    owner = lambda t: t % world
    slot = lambda t: t // world
    arrive = [[[0] * world for _ in range(slots)] for _ in range(world)]      # [owner][slot][sender] = step
    done = [[0] * tiles for _ in range(world)]                                  # [rank][tile] = step
    stage = [[[None] * slots for _ in range(world)] for _ in range(world)]      # [owner][sender][slot] = (step, tile)
    out = [[[None] * tiles for _ in range(2)] for _ in range(world)]            # [rank][buffer][tile] = step
    # per rank: the step its kernel is running (0 = none yet), per CTA a program counter
    cur = [0] * world
    consumed = [0] * world
    ctas = [[None] * grid for _ in range(world)]

    def launch(r):
        cur[r] += 1
        for c in range(grid):
            mine = list(range(c, tiles, grid))
            # phases: one entry per tile, then one "wait for completion flags" entry
            ctas[r][c] = {"tiles": mine, "pc": 0, "final": 0}

    for r in range(world):
        launch(r)
    budget = 200000
    while budget > 0:
        budget -= 1
        if all(cur[r] == steps and consumed[r] == steps for r in range(world)):
            return True
        r = rng.randrange(world)
        s = cur[r]
        live = [c for c in range(grid) if ctas[r][c] is not None]
        if not live:
            # the launch has retired: the consumer reads this step's rows, then the next launch starts
            if consumed[r] < s:
                for t in range(tiles):
                    assert out[r][s & 1][t] == s, f"rank {r} step {s}: tile {t} holds step {out[r][s & 1][t]}"
                consumed[r] = s
            if s < steps:
                launch(r)
            continue
        c = rng.choice(live)
        st = ctas[r][c]
        if st["pc"] < len(st["tiles"]):
            t = st["tiles"][st["pc"]]
            o, k = owner(t), slot(t)
            if o != r:
                stage[o][r][k] = (s, t)          # peer stores of the partial, then the flag
                arrive[o][k][r] = s
                st["pc"] += 1
            else:
                if any(arrive[r][k][q] - s < 0 for q in range(world) if q != r):
                    continue                     # still waiting for a sender
                for q in range(world):
                    if q != r:
                        assert stage[r][q][k] == (s, t), f"owner {r} tile {t} step {s}: staged {stage[r][q][k]}"
                for d in range(world):
                    out[d][s & 1][t] = s         # rows to every rank, then the completion flags
                for d in range(world):
                    if d != r:
                        done[d][t] = s
                st["pc"] += 1
        else:
            waits = [t for t in st["tiles"] if owner(t) != r]
            if st["final"] < len(waits):
                if done[r][waits[st["final"]]] - s < 0:
                    continue
                st["final"] += 1
            else:
                ctas[r][c] = None                # the CTA retires
    return False


@pytest.mark.parametrize("world,grid,tiles", [(2, 4, 10), (2, 6, 6), (4, 6, 20), (8, 12, 40), (3, 5, 17), (8, 4, 3)])
def test_every_schedule_finishes_and_reads_what_it_should(world, grid, tiles):
    for seed in range(40):
        assert run_schedule(world, grid, tiles, steps=4, seed=seed), f"seed {seed}: the ranks wait for each other"


def test_the_model_catches_a_broken_order():
    """The check has teeth: if one rank walked its tiles backwards, owners on different ranks could wait for
    each other's later tiles; the model must then find a schedule that does not finish."""
    def broken(world, grid, tiles, steps, seed):
        # same model, but rank 1's CTAs take their tiles in decreasing order
        rng = random.Random(seed)
        slots = -(-tiles // world)
        arrive = [[[0] * world for _ in range(slots)] for _ in range(world)]
        pcs = [[0] * grid for _ in range(world)]
        order = lambda r, c: (list(range(c, tiles, grid)) if r != 1 else list(range(c, tiles, grid))[::-1])
        for _ in range(20000):
            if all(pcs[r][c] >= len(order(r, c)) for r in range(world) for c in range(grid)):
                return True
            r, c = rng.randrange(world), rng.randrange(grid)
            seq = order(r, c)
            if pcs[r][c] >= len(seq):
                continue
            t = seq[pcs[r][c]]
            o, k = t % world, t // world
            if o != r:
                arrive[o][k][r] = 1
            elif any(arrive[r][k][q] < 1 for q in range(world) if q != r):
                continue
            pcs[r][c] += 1
        return False

    assert run_schedule(2, 1, 4, 1, 0)
    assert not all(broken(2, 1, 4, 1, seed) for seed in range(20))
