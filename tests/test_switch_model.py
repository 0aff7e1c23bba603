"""The in-switch all-reduce's pipeline (csrc/gb_switch.cu) as a CPU model, and its planner.

Model: one block index on every rank of a team.  A rank is a coroutine that runs the kernel's
steps - copy a tile into the own staging buffer, reduce a stripe through the "switch" (read the
stripe in every member's buffer, write the sum into every member's buffer), exchange island
sums through bridge slots, copy a tile out - one memory operation at a time, with the kernel's
one barrier per step (flags with sequence numbers, as sw_block_sync).  A seeded scheduler
interleaves the ranks at random.  Checked on every interleaving: a reduce reads only the
inputs of the tile it reduces, a copy-out reads only finished sums of its tile, nobody reads a
bridge slot of another tile.  The negative control takes one staging buffer away and must be
caught.

Planner: gb_switch_plan's tile and grid keep every buffer inside its region for any size."""
import ctypes
import random

import pytest


class Team:
    def __init__(self, islands, depth, seed):
        self.islands = islands                      # list of lists of ranks
        self.world = sum(len(i) for i in islands)
        self.k = min(len(i) for i in islands)
        self.hier = len(islands) > 1
        self.depth = depth
        self.rng = random.Random(seed)
        self.flags = [[0] * self.world for _ in range(self.world)]      # flags[q][r]: r's last step seen by q
        self.stage = [[[None] * self.k for _ in range(depth)] for _ in range(self.world)]
        self.slots = [[[None] * len(islands) for _ in range(2)] for _ in range(self.world)]
        self.out = [dict() for _ in range(self.world)]
        self.problems = []

    def island_of(self, r):
        for g, members in enumerate(self.islands):
            if r in members:
                return g, members.index(r)
        raise AssertionError

    def barrier(self, r, seq):
        for q in range(self.world):
            if q != r:
                yield
                self.flags[q][r] = seq
        for q in range(self.world):
            while q != r and self.flags[r][q] < seq:
                yield

    def rank(self, r, tiles):
        g, pos = self.island_of(r)
        group = self.islands[g] if self.hier else [x for i in self.islands for x in i]
        owners = self.k if self.hier else self.world
        gpos = pos if self.hier else group.index(r)
        depth, seq = self.depth, 0
        steps = tiles + (4 if self.hier else 3) - 1
        for i in range(steps):
            if i < tiles:                                                    # A: copy in
                for p in range(len(self.stage[r][0])):                      # every stripe of the tile
                    yield
                    self.stage[r][i % depth][p] = ("in", i)
            t = i - 1
            if 0 <= t < tiles and gpos < owners:                             # B: reduce in the switch
                p = gpos
                for m in group:
                    yield
                    got = self.stage[m][t % depth][p]
                    if got != ("in", t):
                        self.problems.append(f"rank {r} reduced tile {t} but member {m} held {got}")
                if not self.hier:
                    for m in group:
                        yield
                        self.stage[m][t % depth][p] = ("sum", t)
                else:
                    for h, members in enumerate(self.islands):
                        yield
                        self.slots[members[pos]][t & 1][g] = ("island", t, g)
            s = i - 2
            if self.hier and 0 <= s < tiles and gpos < owners:               # C: add the islands
                for h in range(len(self.islands)):
                    yield
                    got = self.slots[r][s & 1][h]
                    if got != ("island", s, h):
                        self.problems.append(f"rank {r} added slot {h} of tile {s} but it held {got}")
                for m in group:
                    yield
                    self.stage[m][s % depth][gpos] = ("sum", s)
            c = i - ((4 if self.hier else 3) - 1)
            if c >= 0:                                                       # copy out
                for p in range(len(self.stage[r][0])):
                    yield
                    got = self.stage[r][c % depth][p]
                    if got != ("sum", c):
                        self.problems.append(f"rank {r} copied out tile {c} stripe {p}: {got}")
            if i + 1 < steps:
                seq += 1
                yield from self.barrier(r, seq)

    def run(self, tiles):
        live = [self.rank(r, tiles) for r in range(self.world)]
        while live:
            i = self.rng.randrange(len(live))
            for _ in range(self.rng.choice((1, 1, 3, 10, 40))):
                try:
                    next(live[i])
                except StopIteration:
                    live.pop(i)
                    break
        return self.problems


def _team(islands, depth, seed):
    team = Team(islands, depth, seed)
    if not team.hier:                       # one group: a stripe per member
        team.k = team.world
        team.stage = [[[None] * team.world for _ in range(depth)] for _ in range(team.world)]
    return team


@pytest.mark.parametrize("islands,depth", [([[0, 1]], 3), ([[0, 1, 2, 3]], 3), ([[0, 1], [2, 3]], 4),
                                           ([[0, 1, 2], [3, 4]], 4), ([[0], [1], [2, 3]], 4)])
def test_pipeline_buffers_never_collide(islands, depth):
    for seed in range(40):
        problems = _team(islands, depth, seed).run(tiles=7)
        assert not problems, (seed, problems[:3])


@pytest.mark.parametrize("islands,depth", [([[0, 1, 2]], 2), ([[0, 1], [2, 3]], 3)])
def test_one_buffer_fewer_is_caught(islands, depth):
    seen = any(_team(islands, depth, seed).run(tiles=7) for seed in range(60))
    assert seen, "the model cannot tell a missing staging buffer: it checks nothing"


def test_plan_keeps_every_buffer_inside_its_region():
    from gpubridge_b200.ops import _lib
    lib = _lib.lib()
    rng = random.Random(5)
    for owners, hier, islands in ((8, 0, 1), (2, 0, 1), (4, 1, 2), (2, 1, 4), (3, 1, 2), (1, 1, 2)):
        sw = _lib.GbSwitch()
        sw.bytes, sw.owners, sw.hier = 128 << 20, owners, hier
        sw.len_bridge = (16 << 20) if hier else 0
        depth = 4 if hier else 3
        for _ in range(300):
            nbytes = rng.choice((1, 2, 100, 4096, 8192, 70_000, 1 << 20, (1 << 20) + 2, 37 << 20,
                                 1 << 30, rng.randrange(1, 1 << 31)))
            blocks = rng.choice((1, 8, 32, 128, 160, 500))
            plan = _lib.GbSwitchPlan()
            assert lib.gb_switch_plan(ctypes.byref(sw), islands, nbytes, blocks, ctypes.byref(plan)) == 0
            assert plan.tile % (128 * owners) == 0 and plan.tile > 0
            assert plan.ntiles * plan.tile >= nbytes > (plan.ntiles - 1) * plan.tile
            assert 1 <= plan.grid <= min(2 * blocks, 320, plan.ntiles)      # half-size blocks, two per SM
            assert plan.grid * depth * plan.tile <= sw.bytes
            if hier:
                assert plan.grid * 2 * islands * (plan.tile // owners) <= sw.len_bridge
