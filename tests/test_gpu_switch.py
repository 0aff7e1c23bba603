"""The in-switch all-reduce (csrc/gb_switch.cu) on hardware.

One GPU: a team of one with its own multicast object - the switch "sums" one copy, so the
result is the input (or the input divided), which exercises the tiling, the padding of odd
sizes, the three-buffer pipeline, the per-block barrier numbers across many launches and the
copy stages.  Two or more GPUs: exact sums on integer-valued data for one island (flat order)
and for several (island sums in the switch, islands added over peer memory), identical bits
on every rank, AVG divided once.  All against plain PyTorch sums in fp32."""
import os

import pytest
import torch

from _harness import expected_sum, gpu_ranks, rank_tensor, run_ranks

pytestmark = pytest.mark.gpu

NGPU = torch.cuda.device_count() if torch.cuda.is_available() else 0
WORLD = 8 if NGPU >= 8 else 4 if NGPU >= 4 else 2
SIZES = (1, 17, 4099, 65536 + 3, (1 << 20) + 5, (9 << 20) + 3)


def test_team_of_one_round_trips_through_switch_memory():
    from gpubridge_b200.ops import fabric as fabric_mod
    dev = torch.device("cuda", 0)
    fabric = fabric_mod.create_single(dev)
    try:
        if not fabric.enable_switch():
            pytest.skip(f"this GPU or driver cannot bind multicast memory: {fabric.switch_error}")
        fabric.switch_min_bytes, fabric.switch_min_ranks = 0, 1     # every size takes the switch path
        before = fabric.launches
        for dtype in (torch.float32, torch.bfloat16, torch.float16):
            for n in SIZES + ((40 << 20) + 1,):
                if dtype is not torch.float32 and n > (10 << 20):
                    continue
                x = rank_tensor(3, n, dtype).to(dev)
                out = torch.full_like(x, 7)
                fabric.all_reduce(x, out=out)
                assert torch.equal(out, x), ("sum", dtype, n)
                fabric.all_reduce(x, divide=4, out=out)
                assert torch.equal(out.float(), (x.float() / 4).to(dtype).float()), ("avg", dtype, n)
        # a tensor that lives in switch memory is reduced in place, slices of it too
        home = fabric.switch_empty((3 << 20) + 64)
        assert home is not None and float(home.abs().sum()) == 0.0
        home.copy_(rank_tensor(2, home.numel()).to(dev))
        keep = home.clone()
        fabric.all_reduce(home)
        fabric.all_reduce(home[1024:1024 + 65536], divide=2)
        keep[1024:1024 + 65536] /= 2
        assert torch.equal(home, keep)
        # an unaligned view: the copy stages fall back to narrower accesses
        base = rank_tensor(5, 100_003).to(dev)
        view = base[1:]
        keep = view.clone()
        fabric.all_reduce(view)
        assert torch.equal(view, keep)
        torch.cuda.synchronize(dev)
        fabric.check()
        assert fabric.launches - before >= 2 * 3 * len(SIZES)
    finally:
        torch.cuda.synchronize(dev)
        fabric.close()


def _sums(rank, topology):
    import gpubridge_b200 as gb
    fabric = topology.fabric
    if fabric is None or fabric.sw_team is None:
        return "unavailable: " + (fabric.switch_error if fabric is not None else "no fabric")
    dev, world = topology.device, topology.world_size
    fabric.switch_min_bytes, fabric.switch_min_ranks = 0, 2
    if fabric._engine:
        fabric._engine_switch()
    before = fabric.launches
    for dtype in (torch.float32, torch.bfloat16, torch.float16):
        for n in SIZES:
            t = rank_tensor(rank, n, dtype).to(dev)
            gb.all_reduce(t)
            assert torch.equal(t.cpu(), expected_sum(world, n, dtype)), ("sum", dtype, n)
    for n in (33, 100_003, (3 << 20) + 7):
        t = rank_tensor(rank, n).to(dev)
        gb.all_reduce(t, gb.ReduceOp.AVG)
        assert torch.equal(t.cpu(), expected_sum(world, n) / world), ("avg", n)
    # in place, inside switch memory (what the trainer does with its gradient buffer)
    n = (5 << 20) + 256
    home = fabric.switch_empty(n)
    assert home is not None, fabric.switch_error
    for lo, hi in ((0, n), (4096, 4096 + (1 << 20)), (n - 512, n)):
        home.copy_(rank_tensor(rank, n).to(dev))
        gb.barrier()                                  # nobody reduces while a peer still fills its copy
        torch.cuda.synchronize()
        topology.fabric.all_reduce(home[lo:hi], divide=world)
        torch.cuda.current_stream().wait_stream(topology.fabric.comm_stream)
        want = rank_tensor(rank, n)
        want[lo:hi] = expected_sum(world, n)[lo:hi] / world
        assert torch.equal(home.cpu(), want), ("in place", lo, hi)
        gb.barrier()
        torch.cuda.synchronize()
    # random values: every rank must hold the same bits, close to the fp64 sum
    g = torch.Generator().manual_seed(99 + rank)
    t = torch.randn((2 << 20) + 11, generator=g).to(dev)
    gb.all_reduce(t)
    exact = sum(torch.randn((2 << 20) + 11, generator=torch.Generator().manual_seed(99 + r)).double()
                for r in range(world))
    assert (t.cpu().double() - exact).abs().max() < 1e-4
    rows = torch.empty(world * t.numel(), device=dev)
    gb.all_gather_into_tensor(rows, t)
    rows = rows.view(world, -1)
    assert all(torch.equal(r, rows[0]) for r in rows), "ranks disagree on the bits"
    assert fabric.launches > before
    gb.barrier()
    return "hier" if fabric.sw_island is not None else "flat"


@pytest.mark.skipif(NGPU < 2, reason="needs at least two GPUs")
@pytest.mark.parametrize("split", [{}, {"GPUBRIDGE_SPLIT_TEST": "half"},
                                   {"GPUBRIDGE_SPLIT_TEST": "half", "GPUBRIDGE_SWITCH_FLAT": "0"}]
                         # the hierarchical order on uneven and on four islands has not run on eight
                         # GPUs yet (it has on 2+2): those cases join with GPUBRIDGE_TEST_SWITCH_HIER8=1
                         + ([{"GPUBRIDGE_ISLANDS": "3,5", "GPUBRIDGE_SWITCH_FLAT": "0"},
                             {"GPUBRIDGE_ISLANDS": "2,2,2,2", "GPUBRIDGE_SWITCH_FLAT": "0"}]
                            if WORLD == 8 and os.environ.get("GPUBRIDGE_TEST_SWITCH_HIER8") == "1" else []),
                         ids=lambda s: ",".join(s.values()) or "one-island")
def test_sums_through_the_switch(tmp_path, split):
    # two ranks take the switch only when told to (it saves them no traffic): the kernels are the same
    out = run_ranks(gpu_ranks(WORLD), _sums, tmp_path,
                    env={"GPUBRIDGE_NVLS": "1", "GPUBRIDGE_SWITCH_MIN_RANKS": "2", **split}, timeout=240)
    if any(str(o).startswith("unavailable") for o in out):
        pytest.skip(f"no NVLink multicast binding on this machine ({out[0]})")
    # islands of one GPU cannot have a multicast object of their own: the team's is used
    sizes = {"GPUBRIDGE_SPLIT_TEST": [WORLD // 2], "GPUBRIDGE_ISLANDS": [3, 5] if "3,5" in split.values() else [2]}
    smallest = min(sizes[next(iter(split))]) if split else WORLD
    want = "hier" if split.get("GPUBRIDGE_SWITCH_FLAT") == "0" and smallest >= 2 else "flat"
    assert set(out) == {want}, out


def _copies(rank, topology):
    """Reduce-scatter, all-gather and broadcast through the switch (pieces in multiples of 16
    bytes), every size twice in a row, against the values the collective must produce; sizes
    whose pieces are not multiples of 16 bytes take the peer-memory kernels and must still be
    right."""
    import gpubridge_b200 as gb
    fabric = topology.fabric
    if fabric is None or fabric.sw_team is None:
        return f"unavailable: {getattr(fabric, 'switch_error', 'no fabric')}"
    dev, world = topology.device, topology.world_size
    assert fabric.switch_copy_min_bytes == fabric.switch_gather_min_bytes == 16
    before = fabric.launches
    for dtype in (torch.float32, torch.bfloat16):
        for n in (8, 1024, 70_000, (3 << 20) + 8, 6_000_000, 4099):
            for _ in range(2):
                full = rank_tensor(rank, world * n, dtype).to(dev)
                keep = full.clone()
                out = torch.full((n,), 9, dtype=dtype, device=dev)
                gb.reduce_scatter_tensor(out, full)
                want = expected_sum(world, world * n, dtype).view(world, n)[rank]
                assert torch.equal(out.cpu(), want), ("reduce_scatter", n, dtype)
                assert torch.equal(full, keep), "reduce_scatter must not modify its input"
                if dtype is torch.float32:
                    gb.reduce_scatter_tensor(out, full, gb.ReduceOp.AVG)
                    assert torch.equal(out.cpu(), want / world), ("reduce_scatter avg", n)
                gathered = torch.full((world * n,), 9, dtype=dtype, device=dev)
                gb.all_gather_into_tensor(gathered, rank_tensor(rank, n, dtype).to(dev))
                want = torch.cat([rank_tensor(r, n, dtype) for r in range(world)])
                assert torch.equal(gathered.cpu(), want), ("all_gather", n, dtype)
                for src in (0, world - 1):
                    t = rank_tensor(rank, n, dtype).to(dev)
                    gb.broadcast(t, src)
                    assert torch.equal(t.cpu(), rank_tensor(src, n, dtype)), ("broadcast", n, src)
    torch.cuda.synchronize(dev)
    fabric.check()
    assert fabric.launches > before
    gb.barrier()
    return "ok"


@pytest.mark.skipif(NGPU < 2, reason="needs at least two GPUs")
@pytest.mark.parametrize("split", [{}, {"GPUBRIDGE_SPLIT_TEST": "half"}], ids=["one-island", "half"])
def test_copy_shaped_collectives_through_the_switch(tmp_path, split):
    env = {"GPUBRIDGE_NVLS": "1", "GPUBRIDGE_SWITCH_COPY_MIN_BYTES": "16", "GPUBRIDGE_SWITCH_MIN_RANKS": "2",
           "GPUBRIDGE_SWITCH_GATHER_MIN_BYTES": "16", **split}
    out = run_ranks(gpu_ranks(WORLD), _copies, tmp_path, env=env, timeout=240)
    if any(str(o).startswith("unavailable") for o in out):
        pytest.skip(f"no NVLink multicast binding on this machine ({out[0]})")
    assert set(out) == {"ok"}
