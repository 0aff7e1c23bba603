"""The native engine (csrc/gb_engine.cu) against the Python planner (ops/fabric.py): for the
same team and tensor both must pick the same kernel, grid and arguments - every rank of a
team may be driven by either, and their stripes have to line up.  No GPU: launches are
recorded, not made."""
import ctypes
import random
import threading
import types

import pytest
import torch

from gpubridge_b200.ops import _lib, fabric as fabric_mod

pytestmark = pytest.mark.skipif(not _lib.available(), reason="the native library is not built")

FIELDS = [name for name, _ in _lib.GbArgs._fields_ if name not in ("pad", "residual", "sym", "mc")]


def fake_fabric(sizes, ws_bytes=384 << 20, **over):
    """A Fabric with its planning state but no device: regions carved, launches recorded."""
    f = fabric_mod.Fabric.__new__(fabric_mod.Fabric)
    f.lib = _lib.lib()
    f.world, f.rank = sum(sizes), 0
    f.n_islands, f.k, f.m_max = len(sizes), min(sizes), max(sizes)
    f.ws_bytes = ws_bytes
    f.device, f.comm_stream = torch.device("cpu"), None
    f.max_blocks, f.copy_blocks, f.scatter_blocks, f.overlap_blocks = 128, 32, 64, 32
    f.ring, f.two_shot, f.nvls, f.algo = "phased", False, None, "auto"
    f.force_chunks = f.force_channels = None
    f._caps, f._closed, f._engine, f.launches = threading.local(), False, None, 0
    f.sw_team = f.sw_island = None
    f._heaps = []
    f.switch_min_bytes, f.switch_flat, f.switch_min_ranks = 64 << 10, False, 3
    f.switch_copy_min_bytes, f.switch_gather_min_bytes = 32 << 20, 1 << 62
    f.switch_oneshot_max = min(4 << 20, (16 << 20) // f.world)
    f.layout = types.SimpleNamespace(index=lambda r: r)
    for name, value in over.items():
        setattr(f, name, value)
    team = _lib.GbTeam()
    team.rank, team.world, team.n_islands = 0, f.world, f.n_islands
    position = 0
    for g, size in enumerate(sizes):
        team.island_off[g] = position
        for _ in range(size):
            team.order[position] = position
            position += 1
    team.island_off[len(sizes)] = position
    f.team = team
    f._plan_regions()
    f.seen = []
    f._begin = lambda: None
    f._end = lambda current: None
    f._launch_reduce = lambda kind, dtype, op, codec, args, grid: f.seen.append((0, kind, grid, args))
    f._launch_copy = lambda kind, args, grid: f.seen.append((1, kind, grid, args))
    return f


def same(launch, seen):
    family, kind, grid, args = seen
    assert (launch.family, launch.kind, launch.grid) == (family, kind, grid)
    for name in FIELDS:
        assert getattr(launch.args, name) == getattr(args, name), name


LAYOUTS = [(1,), (2,), (8,), (4, 4), (2, 2, 2, 2), (3, 5), (2, 6), (1, 1), (3, 3, 2)]


@pytest.mark.parametrize("sizes", LAYOUTS)
def test_all_reduce_plans_agree(sizes):
    rng = random.Random(hash(sizes) & 0xFFFF)
    for over in ({}, {"ring": True}, {"ring": False}, {"two_shot": True}, {"algo": "two-shot"},
                 {"force_channels": 2, "force_chunks": 5}, {"max_blocks": 48}):
        f = fake_fabric(sizes, **over)
        engine = f.engine()
        assert engine
        for dtype in (torch.float32, torch.bfloat16, torch.int64, torch.uint8):
            esize = torch.empty(0, dtype=dtype).element_size()
            for _ in range(12):
                n = rng.choice([1, 255, 256, 4097, 1 << 16, (1 << 20) + 3, rng.randrange(1, 1 << 22),
                                rng.randrange(1 << 22, 1 << 26)])
                base = 1 << 30
                inp = base + rng.choice([0, 16, 4, 256]) * 1
                fake = types.SimpleNamespace(
                    numel=lambda n=n: n, nbytes=n * esize, dtype=dtype, data_ptr=lambda inp=inp: inp,
                    element_size=lambda esize=esize: esize)
                cap = rng.choice([0, 0, 32, 7])
                with f.grid_cap(cap or None):
                    f.all_reduce(fake, "sum", divide=f.world)
                launch = _lib.GbLaunch()
                rc = f.lib.gb_engine_prepare_all_reduce(engine, inp, inp, n, _lib.DTYPES[dtype], 0,
                                                        f.world, cap, ctypes.byref(launch))
                assert rc == 0
                same(launch, f.seen.pop())
        f.lib.gb_engine_destroy(engine)


@pytest.mark.parametrize("sizes", [(2,), (8,), (4, 4), (3, 5)])
def test_copy_shaped_plans_agree(sizes):
    rng = random.Random(7)
    f = fake_fabric(sizes)
    engine = f.engine()
    for _ in range(40):
        esize = rng.choice([1, 2, 4, 8])
        dtype = {1: torch.uint8, 2: torch.bfloat16, 4: torch.float32, 8: torch.float64}[esize]
        n = rng.choice([1, 17, 4096, rng.randrange(1, 1 << 24)])
        cap = rng.choice([0, 16])
        small = types.SimpleNamespace(numel=lambda n=n: n, nbytes=n * esize, dtype=dtype, data_ptr=lambda: 4096,
                                      element_size=lambda esize=esize: esize)
        big = types.SimpleNamespace(numel=lambda n=n: n * f.world, nbytes=n * esize * f.world, dtype=dtype,
                                    data_ptr=lambda: 8192, element_size=lambda esize=esize: esize)
        launch = _lib.GbLaunch()
        with f.grid_cap(cap or None):
            f.reduce_scatter(small, big, divide=f.world)
        assert f.lib.gb_engine_prepare_reduce_scatter(engine, 8192, 4096, n, _lib.DTYPES[dtype], f.world, cap,
                                                      ctypes.byref(launch)) == 0
        same(launch, f.seen.pop())
        with f.grid_cap(cap or None):
            f.all_gather(big, small)
        assert f.lib.gb_engine_prepare_all_gather(engine, 4096, 8192, n * esize, cap, ctypes.byref(launch)) == 0
        same(launch, f.seen.pop())
        root = rng.randrange(f.world)
        with f.grid_cap(cap or None):
            f.broadcast(small, root)
        assert f.lib.gb_engine_prepare_broadcast(engine, 4096, n * esize, root, cap, ctypes.byref(launch)) == 0
        same(launch, f.seen.pop())
    f.lib.gb_engine_destroy(engine)


def test_plan_function_matches_and_refuses_small_workspaces():
    rng = random.Random(3)
    L = _lib.lib()
    for _ in range(2000):
        islands = rng.choice([1, 2, 4])
        m_max = rng.choice([1, 2, 4, 8])
        k = rng.randrange(1, m_max + 1)
        esize = rng.choice([1, 2, 4, 8])
        n = rng.randrange(1, 1 << 27)
        stripe_bytes = rng.choice([1 << 16, 1 << 20, 5 << 20]) // 2048 * 2048
        kw = dict(k=k, m_max=m_max, n_islands=islands, len_ha=m_max * stripe_bytes,
                  len_hb=islands * stripe_bytes, len_hc=stripe_bytes, grid=rng.choice([1, 8, 32, 100, 128]),
                  chunk_bytes=rng.choice([None, None, 1 << 20]), force_channels=rng.choice([None, 3]),
                  force_chunks=rng.choice([None, 4]), stripe_multiple=rng.choice([256, 256 * islands]))
        out = _lib.GbHierPlanOut()
        rc = L.gb_plan_hier(n, esize, k, m_max, islands, kw["len_ha"], kw["len_hb"], kw["len_hc"], kw["grid"],
                            kw["chunk_bytes"] or 0, kw["force_channels"] or 0, kw["force_chunks"] or 0,
                            kw["stripe_multiple"], ctypes.byref(out))
        try:
            want = fabric_mod.plan_hier(n, esize, **kw)
        except RuntimeError:
            assert rc == -2
            continue
        assert rc == 0
        assert (out.channels, out.grid, out.stripe, out.nchunks, out.len_a, out.len_b, out.len_c) == (
            want.channels, want.grid, want.stripe, want.nchunks, want.len_a, want.len_b, want.len_c)


class _RecordingLib:
    """The native library with the in-switch launch recorded instead of made (it needs a GPU)."""

    def __init__(self, real, seen) -> None:
        self._real, self._seen = real, seen

    def __getattr__(self, name):
        return getattr(self._real, name)

    def gb_switch_all_reduce(self, team, switch, inp, out, n, dtype, divide, limit, stream):
        self._seen.append((2, switch._obj.hier, limit, inp, out, n, divide))
        return 0

    def gb_switch_all_reduce_oneshot(self, team, switch, inp, out, n, dtype, divide, limit, stream):
        self._seen.append((2, 5, limit, inp, out, n, divide))
        return 0

    def gb_switch_reduce_scatter(self, team, switch, inp, out, n, dtype, divide, limit, stream):
        self._seen.append((2, 2, limit, inp, out, n, divide))
        return 0

    def gb_switch_all_gather(self, team, switch, inp, out, nbytes, limit, stream):
        self._seen.append((2, 3, limit, inp, out, nbytes, 0))
        return 0

    def gb_switch_broadcast(self, team, switch, buffer, nbytes, root, limit, stream):
        self._seen.append((2, 4, limit, None, buffer, nbytes, root))
        return 0


@pytest.mark.parametrize("sizes", [(2,), (3,), (4,), (8,), (4, 4), (2, 2, 2, 2), (1, 1, 1)])
@pytest.mark.parametrize("islands_have_groups", [False, True])
def test_the_in_switch_all_reduce_is_chosen_alike(sizes, islands_have_groups, monkeypatch):
    """Both planners send the same tensors through the switch (sum of floats, from the size and
    team size on), with the same group (the island's when there is one) and the same grid limit;
    everything else takes the kernels it took before."""
    monkeypatch.setattr(torch.cuda, "current_stream",
                        lambda device=None: types.SimpleNamespace(cuda_stream=0))
    monkeypatch.setattr(torch.cuda, "stream", lambda s: __import__("contextlib").nullcontext())
    rng = random.Random(len(sizes) * 131 + sum(sizes))
    f = fake_fabric(sizes)
    f.lib = _RecordingLib(f.lib, f.seen)
    f.sw_team = _lib.GbSwitch()
    f.sw_team.hier = 0
    if islands_have_groups and len(sizes) > 1:
        f.sw_island = _lib.GbSwitch()
        f.sw_island.hier = 1
    engine = f.engine()
    assert engine
    through_switch = 0
    for dtype in (torch.float32, torch.bfloat16, torch.float16, torch.int64):
        esize = torch.empty(0, dtype=dtype).element_size()
        for op in ("sum", "max"):
            for _ in range(10):
                n = rng.choice([256, (64 << 10) // esize - 1, (64 << 10) // esize, 1 << 20,
                                (512 << 10) // esize, (512 << 10) // esize + 1, (2 << 20) // esize,
                                (4 << 20) // esize, rng.randrange(1, 1 << 24)])
                inp = 1 << 30
                fake = types.SimpleNamespace(
                    numel=lambda n=n: n, nbytes=n * esize, dtype=dtype, data_ptr=lambda: inp,
                    element_size=lambda esize=esize: esize)
                cap = rng.choice([0, 32, 7])
                divide = f.world if op == "sum" else 0
                with f.grid_cap(cap or None):
                    f.all_reduce(fake, op, divide=divide)
                launch = _lib.GbLaunch()
                rc = f.lib.gb_engine_prepare_all_reduce(engine, inp, inp, n, _lib.DTYPES[dtype],
                                                        _lib.OPS[op], divide, cap, ctypes.byref(launch))
                assert rc == 0
                seen = f.seen.pop()
                if seen[0] == 2:
                    through_switch += 1
                    _, hier, limit, _, _, count, div = seen
                    assert (launch.family, launch.kind, launch.grid) == (2, hier, limit)
                    assert (launch.args.n, launch.args.divide) == (count, div)
                else:
                    same(launch, seen)
    assert (through_switch > 0) == (sum(sizes) >= f.switch_min_ranks)
    f.lib.gb_engine_destroy(engine)


@pytest.mark.parametrize("sizes", [(2,), (4,), (8,), (4, 4)])
def test_copy_shaped_collectives_take_the_switch_alike(sizes, monkeypatch):
    """Reduce-scatter, all-gather and broadcast go through the team's switch group from the same
    size on in both planners, only with pieces and pointers in multiples of 16 bytes, with the
    same grid limit; below it the peer-memory plans still agree field by field."""
    monkeypatch.setattr(torch.cuda, "current_stream",
                        lambda device=None: types.SimpleNamespace(cuda_stream=0))
    monkeypatch.setattr(torch.cuda, "stream", lambda s: __import__("contextlib").nullcontext())
    rng = random.Random(sum(sizes))
    f = fake_fabric(sizes, ws_bytes=1 << 30, switch_gather_min_bytes=rng.choice([32 << 20, 1 << 62]))
    f.lib = _RecordingLib(f.lib, f.seen)
    f.sw_team = _lib.GbSwitch()
    engine = f.engine()
    assert engine
    world, through = f.world, 0

    def tensor(nbytes, dtype, ptr):
        esize = torch.empty(0, dtype=dtype).element_size()
        return types.SimpleNamespace(numel=lambda: nbytes // esize, nbytes=nbytes, dtype=dtype,
                                     data_ptr=lambda: ptr, element_size=lambda: esize)

    for _ in range(40):
        dtype = rng.choice([torch.float32, torch.bfloat16])
        esize = torch.empty(0, dtype=dtype).element_size()
        piece = rng.choice([4096, (8 << 20) // world, (32 << 20) // world, (64 << 20) // world,
                            (64 << 20) // world + 4, (256 << 20) // world]) // esize * esize
        base = (1 << 30) + rng.choice([0, 0, 0, 4])
        cap = rng.choice([0, 0, 16])
        whole, part = tensor(piece * world, dtype, base), tensor(piece, dtype, (1 << 32) + 256)
        launch = _lib.GbLaunch()
        with f.grid_cap(cap or None):
            f.reduce_scatter(part, whole, divide=world)
        assert f.lib.gb_engine_prepare_reduce_scatter(engine, base, part.data_ptr(), piece // esize,
                                                      _lib.DTYPES[dtype], world, cap, ctypes.byref(launch)) == 0
        seen = f.seen.pop()
        if seen[0] == 2:
            through += 1
            assert (launch.family, launch.kind, launch.grid) == seen[:3] and launch.args.n == seen[5]
        else:
            same(launch, seen)
        with f.grid_cap(cap or None):
            f.all_gather(whole, part)
        assert f.lib.gb_engine_prepare_all_gather(engine, part.data_ptr(), base, piece, cap,
                                                  ctypes.byref(launch)) == 0
        seen = f.seen.pop()
        if seen[0] == 2:
            through += 1
            assert (launch.family, launch.kind, launch.grid) == seen[:3] and launch.args.n == seen[5]
        else:
            same(launch, seen)
        f.layout = types.SimpleNamespace(index=lambda r: r)
        with f.grid_cap(cap or None):
            f.broadcast(whole, 1)
        assert f.lib.gb_engine_prepare_broadcast(engine, base, piece * world, 1, cap, ctypes.byref(launch)) == 0
        seen = f.seen.pop()
        if seen[0] == 2:
            through += 1
            assert (launch.family, launch.kind, launch.grid, launch.args.root) == (*seen[:3], seen[6])
        else:
            same(launch, seen)
    assert (through > 0) == (world >= 3)
    f.lib.gb_engine_destroy(engine)


def test_the_copy_plan_fits_the_switch_memory():
    lib = _lib.lib()
    sw = _lib.GbSwitch()
    sw.bytes = 256 << 20
    for nsub in (1, 3, 4, 8, 16):
        for piece in (16, 4096, 100_000 * 16, 8 << 20, 1 << 30):
            for blocks in (1, 8, 32, 128):
                plan = _lib.GbSwitchPlan()
                assert lib.gb_switch_plan_copy(ctypes.byref(sw), nsub, piece, blocks, ctypes.byref(plan)) == 0
                assert plan.tile % 128 == 0 and plan.tile > 0
                assert 1 <= plan.grid <= min(2 * blocks, _lib.SWITCH_MAX_BLOCKS, plan.ntiles)
                assert plan.grid * 3 * nsub * plan.tile <= sw.bytes
                assert (plan.ntiles - 1) * plan.tile < piece <= plan.ntiles * plan.tile
    sw.bytes = 1 << 16
    assert lib.gb_switch_plan_copy(ctypes.byref(sw), 8, 1 << 20, 128, ctypes.byref(_lib.GbSwitchPlan())) == -1
