"""The data movement of the pipelined all-reduce kernel (csrc/gb_collectives.cu:
allreduce_ring_phased_kernel) as a CPU model, driven by the real planner.

Every rank's four steps - A: spread my stripes over the island's owners; B: owners fold the
island's slots and send the result across islands (to every island, or - two-shot bridge, three
or more islands - sub-stripe h only to island h); C: owners add the islands' parts (two-shot:
finish their own sub-stripe and send it to every island); D: everybody collects the finished
stripes from the island's owners - are restated with the kernel's index arithmetic on integer
arrays, two buffers per region alternating with the chunk, one barrier per iteration, and the
ranks of one iteration run in a random order (their steps touch different buffers, so any order
must do).  The sum must come out exactly for every layout, size and order; a plan whose stripes
do not fit their slots, a wrong owner or sub-stripe mapping, or a buffer reused one iteration too
early shows up as a wrong element."""
import random

import numpy as np
import pytest

from gpubridge_b200.ops.fabric import plan_hier

POISON = -(1 << 40)


def up(v, m):
    return -(-v // m) * m


class Team:
    def __init__(self, sizes):
        self.sizes, self.world, self.islands = sizes, sum(sizes), len(sizes)
        self.k, self.m_max = min(sizes), max(sizes)
        self.island_off = [sum(sizes[:g]) for g in range(len(sizes) + 1)]
        self.where = [(g, p) for g, size in enumerate(sizes) for p in range(size)]     # rank -> (island, pos)

    def rank_of(self, island, pos):
        return self.island_off[island] + pos


def run(sizes, n, two_shot, seed, stripe_bytes=64 << 10, buffers=2):
    team, rng = Team(sizes), random.Random(seed)
    esize = 4
    plan = plan_hier(n, esize, k=team.k, m_max=team.m_max, n_islands=team.islands,
                     len_ha=team.m_max * stripe_bytes, len_hb=team.islands * stripe_bytes, len_hc=stripe_bytes,
                     grid=8, force_channels=1, stripe_multiple=256 * team.islands if two_shot else 256)
    stripe, k, I = plan.stripe, team.k, team.islands
    chunk = stripe * k
    nchunks = -(-n // chunk)
    assert nchunks == plan.nchunks
    cap_a, cap_b, cap_c = plan.len_a // esize, plan.len_b // esize, plan.len_c // esize
    assert team.m_max * stripe <= cap_a and I * stripe <= cap_b and stripe <= cap_c, "a stripe overflows its slot"
    ws = [{"A": np.full((2, cap_a), POISON, np.int64), "B": np.full((2, cap_b), POISON, np.int64),
           "C": np.full((2, cap_c), POISON, np.int64)} for _ in range(team.world)]
    data = [np.random.default_rng(seed * 100 + r).integers(-1000, 1000, n) for r in range(team.world)]
    out = [np.full(n, POISON, np.int64) for _ in range(team.world)]
    depth = 3 if I > 1 else 2
    sub = stripe // I

    def valid(c0, j):
        start = c0 + j * stripe
        return 0 if start >= n else min(stripe, n - start)

    def step_a(r, i):
        g, p = team.where[r]
        c0 = i * chunk
        for j in range(k):
            own, v = team.rank_of(g, j), valid(c0, j)
            slot = ws[own]["A"][i & (buffers - 1)]
            slot[p * stripe:p * stripe + v] = data[r][c0 + j * stripe:c0 + j * stripe + v]
            slot[p * stripe + v:p * stripe + up(v, 256)] = 0

    def step_b(r, c):
        g, p = team.where[r]
        need = up(valid(c * chunk, p), 256)
        if need == 0:
            return
        slots = ws[r]["A"][c & (buffers - 1)]
        total = sum(slots[q * stripe:q * stripe + need] for q in range(team.sizes[g]))
        if I == 1:
            ws[r]["C"][c & (buffers - 1)][:need] = total
        elif two_shot:
            for at in range(0, need, 256):                      # whole 256-value pieces land in one sub-stripe
                h = at // sub
                owner = team.rank_of(h, p)
                ws[owner]["B"][c & (buffers - 1)][g * sub + (at - h * sub):g * sub + (at - h * sub) + 256] = total[at:at + 256]
        else:
            for h in range(I):
                ws[team.rank_of(h, p)]["B"][c & (buffers - 1)][g * stripe:g * stripe + need] = total

    def step_c(r, c):
        g, p = team.where[r]
        need = up(valid(c * chunk, p), 256)
        parts = ws[r]["B"][c & (buffers - 1)]
        if two_shot:
            lo = g * sub
            mine = min(max(need - lo, 0), sub)
            if mine == 0:
                return
            total = sum(parts[h * sub:h * sub + mine] for h in range(I))
            for h in range(I):
                ws[team.rank_of(h, p)]["C"][c & (buffers - 1)][lo:lo + mine] = total
        elif need:
            ws[r]["C"][c & (buffers - 1)][:need] = sum(parts[h * stripe:h * stripe + need] for h in range(I))

    def step_d(r, c):
        g, _ = team.where[r]
        c0 = c * chunk
        for j in range(k):
            v = valid(c0, j)
            out[r][c0 + j * stripe:c0 + j * stripe + v] = ws[team.rank_of(g, j)]["C"][c & (buffers - 1)][:v]

    for i in range(nchunks + depth):
        order = list(range(team.world))
        rng.shuffle(order)
        for r in order:                                          # one iteration; a barrier follows it
            _, p = team.where[r]
            owner = p < k
            if i < nchunks:
                step_a(r, i)
            if owner and 1 <= i and i - 1 < nchunks:
                step_b(r, i - 1)
            if I > 1 and owner and 2 <= i and i - 2 < nchunks:
                step_c(r, i - 2)
            if i >= depth:
                step_d(r, i - depth)
    want = sum(data)
    for r in range(team.world):
        assert np.array_equal(out[r], want), (sizes, n, two_shot, r, int(np.argmax(out[r] != want)))
    return nchunks


SIZES = [1, 255, 256, 257, 4097, 70_001, 300_003]


@pytest.mark.parametrize("sizes", [(2,), (8,), (4, 4), (3, 5), (1, 3), (2, 2, 2, 2)])
def test_every_rank_ends_with_the_sum(sizes):
    for seed, n in enumerate(SIZES):
        run(sizes, n, two_shot=False, seed=seed)


@pytest.mark.parametrize("sizes", [(1, 1, 2), (2, 2, 2, 2), (1, 2, 5), (3, 3, 2)])
def test_two_shot_bridge_ends_with_the_sum(sizes):
    chunks = [run(sizes, n, two_shot=True, seed=seed) for seed, n in enumerate(SIZES)]
    assert max(chunks) >= 3                                      # buffers were reused across chunks


def test_the_model_sees_a_buffer_reused_too_early():
    """Negative control: with one buffer per region instead of two, some order of the ranks
    must give a wrong element."""
    wrong = 0
    for seed in range(12):
        try:
            run((2, 2), 300_003, two_shot=False, seed=seed, stripe_bytes=16 << 10, buffers=1)
        except AssertionError:
            wrong += 1
    assert wrong, "one buffer per region changed nothing: the model checks nothing"
