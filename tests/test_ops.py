"""broadcast, all_gather_into_tensor, reduce_scatter_tensor, barrier, async handles and
argument validation in CPU simulation (reference: tests/test_ops.py, test_broadcast.py)."""
import pytest
import torch

from _harness import LAYOUTS, expected_sum, rank_tensor, run_ranks

POLICIES = ("auto", "flat-gloo", "pipelined-reduce-bridge-broadcast", "sharded-bridge")


def _ops(rank, topology):
    import gpubridge_b200 as gb
    world = topology.world_size
    for n in (1, 5, 1031):
        for src in range(world):
            t = rank_tensor(rank, n)
            gb.broadcast(t, src)
            assert torch.equal(t, rank_tensor(src, n)), ("broadcast", n, src)
        out = torch.empty(world * n)
        gb.all_gather_into_tensor(out, rank_tensor(rank, n))
        assert torch.equal(out, torch.cat([rank_tensor(r, n) for r in range(world)]))
        full = rank_tensor(rank, world * n)
        keep = full.clone()
        out = torch.empty(n)
        gb.reduce_scatter_tensor(out, full)
        assert torch.equal(out, expected_sum(world, world * n).view(world, n)[rank])
        assert torch.equal(full, keep)
        gb.reduce_scatter_tensor(out, full, gb.ReduceOp.AVG)
        assert torch.allclose(out, expected_sum(world, world * n).view(world, n)[rank] / world)
    # async: handles complete in order, futures carry the tensor
    works = [gb.all_reduce(rank_tensor(rank, 100 + i), async_op=True) for i in range(6)]
    for i, w in enumerate(works):
        assert w.wait() is True and w.is_completed() and w.exception() is None
        assert torch.equal(w.get_future().value(), expected_sum(world, 100 + i))
    w = gb.barrier(async_op=True)
    w.wait()
    assert w.get_future().value() is None
    gb.barrier()
    # validation: identical on every rank, before any communication
    with pytest.raises(ValueError, match="contiguous"):
        gb.all_reduce(torch.zeros(4, 4).t())
    with pytest.raises(ValueError, match="doesn't support"):
        gb.all_reduce(torch.zeros(4, dtype=torch.bool))
    with pytest.raises(ValueError, match="AVG needs a floating-point"):
        gb.all_reduce(torch.zeros(4, dtype=torch.int32), gb.ReduceOp.AVG)
    with pytest.raises(ValueError, match="PRODUCT"):
        gb.all_reduce(torch.zeros(4), gb.ReduceOp.PRODUCT)
    with pytest.raises(ValueError, match="src must be"):
        gb.broadcast(torch.zeros(4), world)
    with pytest.raises(ValueError, match="world_size"):
        gb.all_gather_into_tensor(torch.zeros(3), torch.zeros(2))
    with pytest.raises(ValueError, match="SUM and AVG"):
        gb.reduce_scatter_tensor(torch.zeros(1), torch.zeros(world), gb.ReduceOp.MAX)
    with pytest.raises(TypeError):
        gb.all_reduce([1, 2, 3])
    return True


@pytest.mark.parametrize("policy", POLICIES)
def test_every_op_two_islands(tmp_path, policy):
    run_ranks(LAYOUTS["2+2"], _ops, tmp_path, init={"policy": policy},
              env={"GPUBRIDGE_CHUNK_BYTES": "128"})


def test_every_op_uneven_islands(tmp_path):
    run_ranks(LAYOUTS["3+1"], _ops, tmp_path, init={"policy": "sharded-bridge"})


def test_every_op_single_island(tmp_path):
    run_ranks(LAYOUTS["single-vendor"], _ops, tmp_path)


def _three_islands(rank, topology):
    import gpubridge_b200 as gb
    assert [len(i.ranks) for i in topology.layout.islands] == [2, 1, 2]
    assert topology.split_test == "islands" and topology.run_kind == "split-test"
    t = rank_tensor(rank, 777)
    gb.all_reduce(t)
    assert torch.equal(t, expected_sum(5, 777))
    return [i.leader for i in topology.layout.islands]


def test_explicit_island_sizes(tmp_path):
    out = run_ranks(("nvidia",) * 5, _three_islands, tmp_path, env={"GPUBRIDGE_ISLANDS": "2,1,2"})
    assert out == [[0, 2, 3]] * 5


def _config_one(rank, topology):
    """The CPU-simulation acceptance configuration: 4 ranks, two islands, N(0,1) values from
    seed 1234 + rank, 1,024 and 1,048,576 float32 elements, every op, checked against float64."""
    import gpubridge_b200 as gb
    world = topology.world_size
    for n in (1024, 1 << 20):
        values = [torch.randn(n, generator=torch.Generator().manual_seed(1234 + r))
                  for r in range(world)]
        exact = sum(v.double() for v in values)
        t = values[rank].clone()
        gb.all_reduce(t)
        assert (t.double() - exact).abs().max() <= 4 * torch.finfo(torch.float32).eps * \
            sum(v.abs().double() for v in values).max()
        t = values[rank].clone()
        gb.broadcast(t, 0)
        assert torch.equal(t, values[0])
        out = torch.empty(world * n)
        gb.all_gather_into_tensor(out, values[rank])
        assert torch.equal(out, torch.cat(values))
        part = torch.empty(n // world)
        gb.reduce_scatter_tensor(part, values[rank])
        want = exact.view(world, -1)[rank]
        assert (part.double() - want).abs().max() < 1e-5
        gb.barrier()
    return True


def test_cpu_simulation_acceptance_config(tmp_path):
    run_ranks(LAYOUTS["2+2"], _config_one, tmp_path, timeout=180)


def _sharded_twice(rank, topology):
    """A policy that builds its own links can be set up again on the same topology (a benchmark
    racing policies does): the second set of links must not meet the first one's store keys."""
    from gpubridge_b200 import policies
    results = []
    made = []
    for _ in range(3):
        policy = policies.ShardedBridge()
        policy.setup(topology)
        made.append(policy)
        t = rank_tensor(rank, 1000)
        policy.all_reduce(t, topology)
        results.append(torch.equal(t, expected_sum(topology.world_size, 1000)))
    for policy in made:
        policy.close()
    return results


def test_a_link_building_policy_can_be_set_up_again(tmp_path):
    for result in run_ranks(LAYOUTS["2+2"], _sharded_twice, tmp_path):
        assert result == [True, True, True]
