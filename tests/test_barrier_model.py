"""The device-side barrier protocol (csrc/gb_common.cuh: gb_sync) as a CPU model.

Every block of every rank is a coroutine that performs the barrier's memory operations one at
a time - read the generation, arrive, the last arrival stores its sequence number into every
peer's flag row and polls its own row, publishes seq / epoch, resets the arrival counter and
bumps the generation; the others poll the generation - and a seeded scheduler interleaves the
coroutines at random, thousands of different ways.  The data protocol of the collectives rides
on top: before the FIRST barrier of collective e a block writes into the parity-(e & 1) half
of a peer's buffer (the only region written without a barrier in front), after the barrier it
reads what its peers wrote.  Checked on every interleaving:

* nobody leaves barrier k before every block of every rank has arrived at it;
* what a block reads after the barrier is what collective e wrote - never a leftover of
  collective e - 2 in the same half, never an early write of collective e + 2;
* flags and generations only grow; arrival counters return to zero;
* with a rank that never shows up, every wait gives up after its bound, the abort word is
  raised, the failure names the missing peer, and every later barrier returns at once.
"""
import random

import pytest

WAIT_LIMIT = 400          # polls before a wait gives up (the kernel: a globaltimer deadline)


class Rank:
    def __init__(self, world):
        self.grid_arrive = self.grid_gen = self.seq = self.epoch = self.abort = 0
        self.flags = [0] * world              # flags[p]: last sequence number peer p announced here
        self.status = None
        self.buffer = [[None] * world, [None] * world]      # [parity][writer]


class Model:
    def __init__(self, world, blocks, seed, missing=()):
        self.world, self.blocks, self.missing = world, blocks, set(missing)
        self.ranks = [Rank(world) for _ in range(world)]
        self.rng = random.Random(seed)
        self.arrived = {}                     # (rank, barrier number) -> blocks that arrived
        self.problems = []

    # -- the barrier: one yield per memory operation ------------------------------------------------
    def sync(self, r, first, number):
        me = self.ranks[r]
        yield                                                   # __threadfence_system
        gen = me.grid_gen
        yield
        me.grid_arrive += 1                                     # atomicAdd
        last = me.grid_arrive == self.blocks
        self.arrived[(r, number)] = self.arrived.get((r, number), 0) + 1
        yield
        seq = me.seq + 1
        if last:
            for p in range(self.world):                         # one thread per peer, any order
                if p != r:
                    yield
                    assert self.ranks[p].flags[r] <= seq, "a flag went backwards"
                    self.ranks[p].flags[r] = seq                # st.release.sys
            for p in range(self.world):
                if p == r:
                    continue
                polls = 0
                while me.flags[p] < seq:                        # ld.acquire.sys
                    polls += 1
                    if polls > WAIT_LIMIT or me.abort:
                        if not me.abort:
                            me.abort, me.status = 1, ("peer", p, seq)
                        break
                    yield
            yield
            me.seq = seq
            if first:
                me.epoch += 1
            me.grid_arrive = 0
            yield
            me.grid_gen += 1                                    # releases this rank's blocks
        else:
            polls = 0
            while me.grid_gen < gen + 1:
                polls += 1
                if polls > 2 * WAIT_LIMIT * self.world or me.abort:
                    if not me.abort:
                        me.abort, me.status = 1, ("grid", None, seq)
                    break
                yield
        yield
        if me.abort:
            return False
        for q in range(self.world):                             # the safety property of a barrier
            if q not in self.missing and self.arrived.get((q, number), 0) != self.blocks:
                self.problems.append(f"rank {r} left barrier {number} before rank {q} had arrived")
        return True

    # -- a kernel: `barriers` barriers; data written before the first one --------------------------
    def block(self, r, b, kernels, barriers):
        number = 0
        for kernel in range(kernels):
            me = self.ranks[r]
            parity = me.epoch & 1                               # read at kernel start, as the kernels do
            epoch = kernel                                      # what this collective is, for the check
            if me.epoch != kernel and not me.abort:
                self.problems.append(f"rank {r} block {b}: epoch {me.epoch} at the start of kernel {kernel}")
            if b == 0:                                          # one writer per rank is enough
                for p in range(self.world):
                    yield
                    self.ranks[p].buffer[parity][r] = (epoch, r)
            for k in range(barriers):
                ok = yield from self.sync(r, k == 0, number)
                number += 1
                if not ok:
                    return
                if k == 0:
                    for w in range(self.world):                 # read what every peer wrote
                        yield
                        got = me.buffer[parity][w]
                        if got != (epoch, w):
                            self.problems.append(f"rank {r} block {b} kernel {kernel}: read {got} from {w}")

    def run(self, kernels, barriers):
        live = [self.block(r, b, kernels, barriers) for r in range(self.world) if r not in self.missing
                for b in range(self.blocks)]
        steps = 0
        while live:
            i = self.rng.randrange(len(live))
            # bursts: a coroutine usually runs several operations before another is scheduled
            for _ in range(self.rng.choice((1, 1, 2, 5, 20))):
                try:
                    next(live[i])
                except StopIteration:
                    live.pop(i)
                    break
            steps += 1
            assert steps < 5_000_000, "the model did not terminate: a wait without a bound"
        return self.problems


@pytest.mark.parametrize("world,blocks,barriers", [(2, 1, 1), (2, 3, 3), (4, 2, 2), (8, 2, 1), (3, 4, 4)])
def test_barrier_and_buffer_parity_under_random_interleavings(world, blocks, barriers):
    for seed in range(60):
        model = Model(world, blocks, seed)
        problems = model.run(kernels=5, barriers=barriers)
        assert not problems, (seed, problems[:3])
        for rank in model.ranks:
            assert rank.grid_arrive == 0 and rank.abort == 0
            assert rank.seq == 5 * barriers and rank.epoch == 5 and rank.grid_gen == 5 * barriers
            assert all(f == rank.seq for p, f in enumerate(rank.flags) if model.ranks[p] is not rank)


def test_one_buffer_half_is_not_enough():
    """The negative control: with a single half (no parity) a fast rank's write for collective
    e + 1 lands while a slow rank still reads collective e - the model must see it."""
    seen = False
    for seed in range(200):
        model = Model(3, 2, seed)
        for rank in model.ranks:
            rank.buffer[1] = rank.buffer[0]          # both parities alias one buffer
        seen = seen or bool(model.run(kernels=4, barriers=1))
    assert seen, "the model cannot tell one buffer half from two: it checks nothing"


@pytest.mark.parametrize("missing", [1, 3])
def test_a_missing_rank_ends_every_wait(missing):
    for seed in range(20):
        model = Model(4, 2, seed, missing=(missing,))
        problems = model.run(kernels=3, barriers=2)
        assert not problems
        for r, rank in enumerate(model.ranks):
            if r == missing:
                continue
            assert rank.abort == 1 and rank.status[0] in ("peer", "grid")
            if rank.status[0] == "peer":
                assert rank.status[1] == missing
            # the failed barrier still publishes its number (as the kernel does); nothing follows it
            assert rank.seq <= 1 and rank.epoch <= 1


# ---- pull-style collectives: stage the own piece, meet, read every peer's staging area ----------
# The all-gather (csrc/gb_collectives.cu: allgather_kernel) leaves without a closing barrier, and
# the all-gather fused into the GEMM (csrc/gb_gemm.cu) stages into the same region.  A rank that
# has finished the all-gather may launch the GEMM and stage its weight shard while a slower peer
# is still pulling the all-gather's piece out of that rank's memory - unless the two collectives
# use different halves of the region, which the parity of the collective counter guarantees.
def _pull_block(model, r, b, kernels, half_of):
    number = 0
    for kernel in range(kernels):
        me = model.ranks[r]
        half = half_of(kernel, me.epoch)                      # read at kernel start
        if b == 0:
            yield
            me.buffer[half][r] = (kernel, r)                    # stage the own piece locally
        ok = yield from model.sync(r, True, number)
        number += 1
        if not ok:
            return
        for p in range(model.world):                            # pull from every peer's memory
            yield
            got = model.ranks[p].buffer[half][p]
            if got != (kernel, p):
                model.problems.append(f"rank {r} block {b} collective {kernel}: pulled {got} from {p}")
        if kernel % 2 == 1:                                     # the fused GEMM closes with a barrier
            ok = yield from model.sync(r, False, number)
            number += 1
            if not ok:
                return


def _run_pull(world, blocks, seed, half_of, kernels=6):
    model = Model(world, blocks, seed)
    live = [_pull_block(model, r, b, kernels, half_of) for r in range(world) for b in range(blocks)]
    while live:
        i = model.rng.randrange(len(live))
        for _ in range(model.rng.choice((1, 1, 2, 5, 20))):
            try:
                next(live[i])
            except StopIteration:
                live.pop(i)
                break
    return model.problems


@pytest.mark.parametrize("world,blocks", [(2, 1), (3, 2), (8, 1)])
def test_all_gather_then_fused_gemm_stage_into_different_halves(world, blocks):
    """Collectives alternate: all-gather (even), fused all-gather GEMM (odd).  Both pick the
    staging half from the collective counter's parity, so the GEMM's staging never lands in the
    half a slow peer is still pulling the all-gather from."""
    for seed in range(60):
        problems = _run_pull(world, blocks, seed, lambda kernel, epoch: epoch & 1)
        assert not problems, (seed, problems[:3])


def test_fused_gemm_always_staging_into_the_first_half_is_caught():
    """The negative control: the GEMM staging into half 0 whatever the counter says (and the
    all-gather before it having used half 0 too) corrupts a slow peer's all-gather."""
    def half_of(kernel, epoch):
        return 0 if kernel % 2 == 1 else epoch & 1
    seen = any(_run_pull(3, 1, seed, half_of, kernels=8) for seed in range(300))
    assert seen, "the model cannot see a staging area overwritten under a slow reader"
