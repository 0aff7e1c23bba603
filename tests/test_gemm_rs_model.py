"""The tile schedule and the addressing of the fused GEMM + reduce-scatter kernel
(csrc/gb_gemm_rs.cu) restated on the CPU: every rank walks its tiles in the kernel's order and
stores each row of its product into the owner's staging area at the kernel's offsets; owners
then add their slots.  Checks that the rotated walk visits every tile once and ends on the own
rows, that no two writers touch the same staging byte, that a collective stays inside its
parity half, and that the result is the averaged product's rows."""
import numpy as np
import pytest

BM, BN = 128, 256


def tiles_in_order(rank, rows_per_rank, P, Q):
    p_tiles, q_tiles = -(-P // BM), -(-Q // BN)
    first = (-(-(rank + 1) * rows_per_rank // BM)) % p_tiles
    for t in range(p_tiles * q_tiles):
        yield ((first + t // q_tiles) % p_tiles) * BM, (t % q_tiles) * BN


@pytest.mark.parametrize("world,P,Q", [(1, 256, 512), (2, 512, 264), (8, 2816, 1024), (4, 384, 72), (8, 1024, 256)])
def test_schedule_and_addressing(world, P, Q):
    rng = np.random.default_rng(P + Q + world)
    rows = P // world
    slot = rows * Q                                   # elements (the kernel: * 2 bytes)
    half = world * slot + 64                          # the region's half is at least world slots
    products = [rng.integers(-50, 50, (P, Q)) for _ in range(world)]
    for parity in (0, 1):
        staging = [np.full(2 * half, -10**9, np.int64) for _ in range(world)]
        written = [np.zeros(2 * half, bool) for _ in range(world)]
        for rank in range(world):
            seen, order = set(), []
            for p0, q0 in tiles_in_order(rank, rows, P, Q):
                assert (p0, q0) not in seen
                seen.add((p0, q0))
                order.append(p0)
                row = p0
                while row < min(p0 + BM, P):                      # the tile's rows, owner by owner
                    owner, at = divmod(row, rows)
                    count = min(rows - at, min(p0 + BM, P) - row)
                    base = parity * half + rank * slot             # the kernel: + at * Q + col per row
                    cols = slice(q0, min(q0 + BN, Q))
                    mark = written[owner][base:base + slot].reshape(rows, Q)
                    data = staging[owner][base:base + slot].reshape(rows, Q)
                    assert not mark[at:at + count, cols].any(), "two writers on one staging element"
                    mark[at:at + count, cols] = True
                    data[at:at + count, cols] = products[rank][row:row + count, cols]
                    row += count
            assert len(seen) == -(-P // BM) * -(-Q // BN)
            if world > 1 and rows % BM == 0:
                own = [p0 for p0 in order if rank * rows <= p0 < (rank + 1) * rows]
                assert order[-len(own):] == own, "the own rows must come last"
        for owner in range(world):
            assert not written[owner][(1 - parity) * half:(2 - parity) * half].any(), "wrote into the other half"
            got = sum(staging[owner][parity * half + s * slot:parity * half + (s + 1) * slot] for s in range(world))
            want = sum(products)[owner * rows:(owner + 1) * rows].reshape(-1)
            assert np.array_equal(got, want)
