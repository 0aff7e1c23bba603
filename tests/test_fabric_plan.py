"""The hierarchical all-reduce plan is pure arithmetic: checked here without a GPU.  Every
stripe must fit its slot in every region for every channel count and team shape, buffers of
neighbouring channels must not overlap, and the plan may only depend on values all ranks
share (two faults of exactly these kinds were found on hardware; these are their guards)."""
import itertools

import pytest

from gpubridge_b200.ops.fabric import plan_hier

MIB = 1 << 20


def _regions(world, m_max, n_islands, ws_bytes=384 * MIB):
    """The carve Fabric._plan_regions makes, restated."""
    slot = max(MIB, min(8 * MIB, 16 * MIB // max(1, world)))
    rest = ws_bytes - 4096 - 2 * world * slot
    hier = rest * 45 // 100
    stripe_bytes = hier // (2 * (m_max + n_islands + 1)) // 2048 * 2048
    return m_max * stripe_bytes, n_islands * stripe_bytes, stripe_bytes


SHAPES = [(1, [1]), (2, [2]), (2, [1, 1]), (4, [2, 2]), (4, [1, 3]), (8, [8]), (8, [4, 4]),
          (8, [3, 5]), (8, [2, 2, 2, 2]), (16, [8, 8])]


@pytest.mark.parametrize("world,islands", SHAPES)
def test_stripes_fit_their_slots(world, islands):
    m_max, k, n_islands = max(islands), min(islands), len(islands)
    len_ha, len_hb, len_hc = _regions(world, m_max, n_islands)
    for esize, nbytes, grid, channels in itertools.product(
            (1, 2, 4, 8), (4096, 3 * MIB + 12, 36 * MIB + 12, 256 * MIB, 1 << 30), (8, 32, 128),
            (None, 1, 2, 4, 8)):
        n = nbytes // esize
        plan = plan_hier(n, esize, k=k, m_max=m_max, n_islands=n_islands, len_ha=len_ha,
                         len_hb=len_hb, len_hc=len_hc, grid=grid, force_channels=channels)
        sbytes = plan.stripe * esize
        assert plan.stripe % 256 == 0 and plan.stripe > 0
        assert m_max * sbytes <= plan.len_a, "an island member's slot leaves region A's buffer"
        assert n_islands * sbytes <= plan.len_b and sbytes <= plan.len_c
        # channel c uses [c * 2 * len, (c + 1) * 2 * len) of each region (two buffers)
        assert plan.channels * 2 * plan.len_a <= 2 * len_ha
        assert plan.channels * 2 * plan.len_b <= 2 * len_hb
        assert plan.channels * 2 * plan.len_c <= 2 * len_hc
        assert plan.grid % plan.channels == 0 and plan.grid >= plan.channels
        assert plan.nchunks * plan.stripe * k >= n
        assert plan.len_a % 4096 == 0 and plan.len_b % 4096 == 0 and plan.len_c % 4096 == 0


def test_plan_does_not_depend_on_the_callers_island():
    """Ranks of a 3-member and of a 5-member island compute the plan from the same inputs: the
    function takes no per-rank argument at all."""
    import inspect
    names = set(inspect.signature(plan_hier).parameters)
    assert not names & {"rank", "my_island", "my_pos", "members", "island_size"}
    len_ha, len_hb, len_hc = _regions(8, 5, 2)
    a = plan_hier(6291457, 2, k=3, m_max=5, n_islands=2, len_ha=len_ha, len_hb=len_hb,
                  len_hc=len_hc, grid=128)
    b = plan_hier(6291457, 2, k=3, m_max=5, n_islands=2, len_ha=len_ha, len_hb=len_hb,
                  len_hc=len_hc, grid=128)
    assert a == b


def test_small_workspace_is_refused():
    with pytest.raises(RuntimeError, match="too small"):
        plan_hier(1 << 20, 4, k=1, m_max=8, n_islands=1, len_ha=8192, len_hb=8192, len_hc=1024,
                  grid=128)


def test_two_shot_stripes_split_evenly_over_the_islands():
    for world, islands in ((8, [2, 2, 2, 2]), (8, [1, 2, 5]), (4, [1, 1, 2])):
        m_max, k, n_islands = max(islands), min(islands), len(islands)
        len_ha, len_hb, len_hc = _regions(world, m_max, n_islands)
        for nbytes in (3 * MIB + 12, 36 * MIB + 12, 1 << 30):
            plan = plan_hier(nbytes // 4, 4, k=k, m_max=m_max, n_islands=n_islands, len_ha=len_ha,
                             len_hb=len_hb, len_hc=len_hc, grid=128,
                             stripe_multiple=256 * n_islands)
            assert plan.stripe % (256 * n_islands) == 0
            assert m_max * plan.stripe * 4 <= plan.len_a and plan.stripe * 4 <= plan.len_c
