"""The copy-shaped collectives through the switch (switch_copy_kernel) as a CPU model.

One block index on every rank.  Depth-3 staging buffers, one barrier at the end of EVERY step
(the last one too).  Per step s: reduce-scatter stages tile s of the input locally and, for
tile s-1, reads the own sub-tile in EVERY member's buffer; all-gather writes its sub-tile of
tile s into EVERY member's buffer and copies tile s-1 out of its own; broadcast is the
all-gather with one writer.  A seeded scheduler interleaves the ranks one memory operation at
a time, and kernels follow one another with no host synchronisation.  Checked on every
interleaving: every read sees exactly the tile it is meant to see, also across the boundary
between two kernels.  (With a barrier after every step two buffers would already do; the third
is slack the kernel shares with the all-reduce's rotation.)  Negative controls: one buffer, and
no barrier after the last step, must both be caught."""
import random

import pytest


class Team:
    def __init__(self, world, seed, depth=3, final_barrier=True):
        self.world, self.depth, self.final_barrier = world, depth, final_barrier
        self.rng = random.Random(seed)
        self.flags = [[0] * world for _ in range(world)]
        # stage[r][buffer][sub-tile] = (kernel, tile) whose data it holds
        self.stage = [[[None] * world for _ in range(depth)] for _ in range(world)]
        self.problems = []

    def barrier(self, r, seq):
        for q in range(self.world):
            if q != r:
                yield
                self.flags[q][r] = seq
        for q in range(self.world):
            while q != r and self.flags[r][q] < seq:
                yield

    def rank(self, r, kernels):
        seq = 0
        for k, (mode, tiles) in enumerate(kernels):
            root = k % self.world
            for s in range(tiles + 1):
                now, before = s % self.depth, (s - 1) % self.depth
                if mode == "reduce_scatter":
                    if s < tiles:
                        for q in range(self.world):               # stage every member's piece, locally
                            yield
                            self.stage[r][now][q] = (k, s)
                    if s >= 1:
                        for q in self.rng.sample(range(self.world), self.world):   # the switch pulls
                            yield
                            if self.stage[q][before][r] != (k, s - 1):
                                self.problems.append(("rs", r, k, s - 1, q, self.stage[q][before][r]))
                else:
                    writer = mode == "all_gather" or r == root
                    slot = r if mode == "all_gather" else 0
                    if s < tiles and writer:
                        for q in self.rng.sample(range(self.world), self.world):   # one store, every member
                            yield
                            self.stage[q][now][slot] = (k, s)
                    if s >= 1 and (mode == "all_gather" or r != root):
                        for q in (range(self.world) if mode == "all_gather" else [0]):
                            yield
                            if self.stage[r][before][q] != (k, s - 1):
                                self.problems.append((mode, r, k, s - 1, q, self.stage[r][before][q]))
                if s < tiles or self.final_barrier:
                    seq += 1
                    yield from self.barrier(r, seq)

    def run(self, kernels):
        live = [self.rank(r, kernels) for r in range(self.world)]
        while live:
            g = self.rng.choice(live)
            try:
                next(g)
            except StopIteration:
                live.remove(g)
        return self.problems


PROGRAMS = {
    "reduce-scatters": [("reduce_scatter", 5), ("reduce_scatter", 1), ("reduce_scatter", 4)],
    "all-gathers": [("all_gather", 4), ("all_gather", 1), ("all_gather", 3)],
    "broadcasts": [("broadcast", 3), ("broadcast", 1), ("broadcast", 4), ("broadcast", 2)],
    "mixed": [("all_gather", 2), ("reduce_scatter", 3), ("broadcast", 2), ("all_gather", 1),
              ("reduce_scatter", 1)],
}


@pytest.mark.parametrize("world", [2, 3, 4, 8])
@pytest.mark.parametrize("name", sorted(PROGRAMS))
def test_every_read_sees_its_own_tile(world, name):
    for seed in range(60):
        assert Team(world, seed).run(PROGRAMS[name]) == [], (world, name, seed)


@pytest.mark.parametrize("name", ["all-gathers", "reduce-scatters"])
def test_a_single_buffer_is_caught(name):
    assert sum(bool(Team(4, seed, depth=1).run(PROGRAMS[name])) for seed in range(200)) > 0


@pytest.mark.parametrize("name", sorted(PROGRAMS))
def test_two_buffers_would_do(name):
    for seed in range(40):
        assert Team(4, seed, depth=2).run(PROGRAMS[name]) == []


def test_a_missing_last_barrier_is_caught():
    # without the barrier after the last step the next kernel's first remote write can land in a
    # buffer a slower member still copies out of
    assert sum(bool(Team(4, seed, final_barrier=False).run(PROGRAMS["all-gathers"]))
               for seed in range(300)) > 0
