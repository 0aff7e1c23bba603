"""The one-step in-switch all-reduce's slot protocol (allreduce_switch_oneshot_kernel) as a CPU model.

One block index on every rank of a team.  A call is: write the own input into half
``seq & 1`` of the own slot, one barrier with the same block of every other rank (flags with
sequence numbers, as sw_block_sync), then read that half of EVERY rank's slot; there is no
barrier after the reads.  Calls follow one another with no host synchronisation, and other
kernels that only run barriers may come in between (a pipelined all-reduce through the same
block index).  A seeded scheduler interleaves the ranks one memory operation at a time.
Checked on every interleaving: a read never sees another call's data - i.e. nobody overwrites a
half that a slower peer still has to read.  The negative control uses one half only and must
be caught."""
import random

import pytest


class Team:
    def __init__(self, world, seed, halves=2):
        self.world, self.halves = world, halves
        self.rng = random.Random(seed)
        self.flags = [[0] * world for _ in range(world)]        # flags[q][r]: r's last barrier seen by q
        self.slot = [[None] * 2 for _ in range(world)]           # slot[r][half]: the call whose data it holds
        self.problems = []

    def barrier(self, r, seq):
        for q in range(self.world):
            if q != r:
                yield
                self.flags[q][r] = seq
        for q in range(self.world):
            while q != r and self.flags[r][q] < seq:
                yield

    def rank(self, r, program):
        seq = 0
        for call, kind in enumerate(program):
            if kind == "barriers":                               # another kernel: two barriers, no slot traffic
                for _ in range(2):
                    seq += 1
                    yield from self.barrier(r, seq)
                continue
            seq += 1
            half = seq % self.halves
            yield
            self.slot[r][half] = call                            # copy in
            yield from self.barrier(r, seq)
            for q in self.rng.sample(range(self.world), self.world):   # the switch pulls from everyone
                yield
                if self.slot[q][half] != call:
                    self.problems.append((r, call, q, self.slot[q][half]))

    def run(self, program):
        live = [self.rank(r, program) for r in range(self.world)]
        while live:
            g = self.rng.choice(live)
            try:
                next(g)
            except StopIteration:
                live.remove(g)
        return self.problems


PROGRAMS = [["one"] * 12,
            ["one", "barriers", "one", "one", "barriers", "barriers", "one", "one", "one"],
            ["barriers", "one", "barriers", "one", "barriers", "one", "one"]]


@pytest.mark.parametrize("world", [2, 3, 4, 8])
@pytest.mark.parametrize("program", PROGRAMS, ids=["back-to-back", "mixed", "alternating"])
def test_nobody_overwrites_what_a_peer_still_reads(world, program):
    for seed in range(150):
        assert Team(world, seed).run(program) == [], (world, seed)


@pytest.mark.parametrize("world", [2, 4])
def test_a_single_half_is_caught(world):
    caught = sum(bool(Team(world, seed, halves=1).run(PROGRAMS[0])) for seed in range(150))
    assert caught > 0
