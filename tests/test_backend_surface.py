"""The surface of ``backend="gpubridge"`` scenario by scenario, on four CPU ranks in two
simulated islands (ranks 0-1 and 2-3) that join ONCE for the whole module (``RankPool``):
every form of every collective torch.distributed offers, the refusals, object collectives,
subgroups, async handles, observers.  Values are integer-valued, so sums are exact in any
order and every check is ``torch.equal``.  (Scenarios follow what the reference's backend
tests cover - tests/test_torch_backend.py - one function per behaviour.)"""
import pytest
import torch

from _harness import TWO_BY_TWO, RankPool

WORLD = 4


@pytest.fixture(scope="module")
def ranks(tmp_path_factory):
    pool = RankPool(TWO_BY_TWO, tmp_path_factory.mktemp("backend-pool"), mode="backend")
    yield pool
    pool.close()


def _values(rank, n=6, dtype=torch.float32):
    return (torch.arange(n) % 5 + rank).to(dtype)


def _total(n=6, dtype=torch.float32):
    return sum(_values(r, n, torch.float64) for r in range(WORLD)).to(dtype)


# ---- all_reduce -----------------------------------------------------------------------------------------
def _all_reduce_ops(rank, world):
    import torch.distributed as dist
    for dtype in (torch.float32, torch.float64, torch.bfloat16, torch.int32, torch.int64, torch.uint8):
        t = _values(rank, 33, dtype)
        dist.all_reduce(t)
        assert torch.equal(t, _total(33, dtype)), dtype
    t = _values(rank)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    assert torch.equal(t, _values(world - 1))
    t = _values(rank)
    dist.all_reduce(t, op=dist.ReduceOp.MIN)
    assert torch.equal(t, _values(0))
    t = _values(rank)
    dist.all_reduce(t, op=dist.ReduceOp.AVG)
    assert torch.equal(t, _total() / world)
    return True


def test_all_reduce_every_op_and_dtype(ranks):
    ranks.run(_all_reduce_ops)


def _avg_of_integers_is_refused(rank, world):
    import torch.distributed as dist
    with pytest.raises((ValueError, RuntimeError, NotImplementedError)):
        dist.all_reduce(torch.ones(4, dtype=torch.int32), op=dist.ReduceOp.AVG)
    dist.barrier()
    return True


def test_avg_of_integers_is_refused_before_any_communication(ranks):
    ranks.run(_avg_of_integers_is_refused)


def _product_and_bitwise(rank, world):
    import torch.distributed as dist
    for op in (dist.ReduceOp.PRODUCT, dist.ReduceOp.BAND, dist.ReduceOp.BOR, dist.ReduceOp.BXOR):
        with pytest.raises(ValueError, match="SUM"):
            dist.all_reduce(torch.ones(2, dtype=torch.int32), op=op)
    t = torch.ones(2)
    dist.all_reduce(t)                       # and the group still works
    assert float(t[0]) == world
    return True


def test_unsupported_reduce_ops_name_the_supported_ones(ranks):
    ranks.run(_product_and_bitwise)


def _all_reduce_coalesced(rank, world):
    import torch.distributed as dist
    a, b, c = _values(rank, 3), _values(rank, 10), _values(rank, 7, torch.float64)
    with dist._coalescing_manager(device=torch.device("cpu"), async_ops=True) as batch:
        for t in (a, b, c):
            dist.all_reduce(t)
    batch.wait()
    assert torch.equal(a, _total(3)) and torch.equal(b, _total(10))
    assert torch.equal(c, _total(7, torch.float64))
    a = _values(rank, 5)
    with dist._coalescing_manager(device=torch.device("cpu")):       # synchronous form
        dist.all_reduce(a)
    assert torch.equal(a, _total(5))
    return True


def test_coalesced_all_reduce_sync_and_async(ranks):
    ranks.run(_all_reduce_coalesced)


def _async_handles(rank, world):
    import torch.distributed as dist
    tensors = [_values(rank, 4 + i) for i in range(6)]
    works = [dist.all_reduce(t, async_op=True) for t in tensors]
    for i, (work, t) in enumerate(zip(works, tensors)):
        assert work.wait() is True
        assert work.is_completed() and work.is_success()
        assert torch.equal(t, _total(4 + i))
        future = work.get_future()
        future.wait()
        assert torch.equal(future.value()[0], _total(4 + i))
    return True


def test_async_handles_complete_in_order_and_carry_the_result(ranks):
    ranks.run(_async_handles)


def _noncontiguous_is_refused(rank, world):
    import torch.distributed as dist
    strided = torch.ones(4, 4)[:, 0]
    with pytest.raises((ValueError, RuntimeError), match="contiguous"):
        dist.all_reduce(strided)
    dist.barrier()
    return True


def test_a_strided_tensor_is_refused(ranks):
    ranks.run(_noncontiguous_is_refused)


# ---- broadcast ----------------------------------------------------------------------------------------
def _broadcast_from_every_rank(rank, world):
    import torch.distributed as dist
    for src in range(world):
        for dtype in (torch.float32, torch.int64, torch.uint8):
            t = _values(rank, 9, dtype)
            dist.broadcast(t, src=src)
            assert torch.equal(t, _values(src, 9, dtype)), (src, dtype)
    with pytest.raises(ValueError, match="doesn't support torch.bool"):      # refused, with the list
        dist.broadcast(torch.ones(3, dtype=torch.bool), src=0)
    work = dist.broadcast(t := _values(rank, 5), src=3, async_op=True)
    work.wait()
    assert torch.equal(t, _values(3, 5))
    return True


def test_broadcast_from_every_rank(ranks):
    ranks.run(_broadcast_from_every_rank)


def _broadcast_object_list(rank, world):
    import torch.distributed as dist
    items = [{"step": 7, "from": rank}, "text", None] if rank == 1 else [None, None, None]
    dist.broadcast_object_list(items, src=1)
    assert items == [{"step": 7, "from": 1}, "text", None]
    return True


def test_broadcast_object_list(ranks):
    ranks.run(_broadcast_object_list)


# ---- all_gather ---------------------------------------------------------------------------------------
def _all_gather_forms(rank, world):
    import torch.distributed as dist
    mine = _values(rank, 5)
    flat = torch.empty(world * 5)
    dist.all_gather_into_tensor(flat, mine)
    assert torch.equal(flat, torch.cat([_values(r, 5) for r in range(world)]))
    stacked = torch.empty(world, 5)
    dist.all_gather_into_tensor(stacked, mine)
    assert torch.equal(stacked, torch.stack([_values(r, 5) for r in range(world)]))
    parts = [torch.empty(5) for _ in range(world)]
    dist.all_gather(parts, mine)
    assert all(torch.equal(p, _values(r, 5)) for r, p in enumerate(parts))
    work = dist.all_gather_into_tensor(flat.zero_(), mine, async_op=True)
    work.wait()
    assert torch.equal(flat, torch.cat([_values(r, 5) for r in range(world)]))
    return True


def test_all_gather_flat_stacked_list_and_async(ranks):
    ranks.run(_all_gather_forms)


def _all_gather_coalesced(rank, world):
    import torch.distributed as dist
    a_out, b_out = torch.empty(world * 3), torch.empty(world * 8, dtype=torch.float64)
    with dist._coalescing_manager(device=torch.device("cpu"), async_ops=True) as batch:
        dist.all_gather_into_tensor(a_out, _values(rank, 3))
        dist.all_gather_into_tensor(b_out, _values(rank, 8, torch.float64))
    batch.wait()
    assert torch.equal(a_out, torch.cat([_values(r, 3) for r in range(world)]))
    assert torch.equal(b_out, torch.cat([_values(r, 8, torch.float64) for r in range(world)]))
    return True


def test_coalesced_all_gather_into_tensor(ranks):
    ranks.run(_all_gather_coalesced)


def _all_gather_object(rank, world):
    import torch.distributed as dist
    seen = [None] * world
    dist.all_gather_object(seen, {"rank": rank, "blob": "x" * (10 + 100 * rank)})
    assert [s["rank"] for s in seen] == list(range(world))
    assert [len(s["blob"]) for s in seen] == [10 + 100 * r for r in range(world)]
    kept = [None] * world if rank == 2 else None
    dist.gather_object(rank * rank, kept, dst=2)
    assert kept == ([0, 1, 4, 9] if rank == 2 else None)
    got = [None]
    dist.scatter_object_list(got, [f"for {r}" for r in range(world)] if rank == 0 else None, src=0)
    assert got == [f"for {rank}"]
    return True


def test_object_collectives(ranks):
    ranks.run(_all_gather_object)


# ---- reduce_scatter -----------------------------------------------------------------------------------
def _reduce_scatter_forms(rank, world):
    import torch.distributed as dist
    full = _values(rank, world * 4)
    keep = full.clone()
    out = torch.empty(4)
    dist.reduce_scatter_tensor(out, full)
    assert torch.equal(out, _total(world * 4).view(world, 4)[rank])
    assert torch.equal(full, keep), "the input must come back untouched"
    dist.reduce_scatter_tensor(out, full, op=dist.ReduceOp.AVG)
    assert torch.equal(out, (_total(world * 4) / world).view(world, 4)[rank])
    with pytest.raises(ValueError, match="SUM and AVG"):
        dist.reduce_scatter_tensor(out, full, op=dist.ReduceOp.MAX)
    out = torch.empty(4)
    dist.reduce_scatter(out, list(full.view(world, 4).unbind(0)))
    assert torch.equal(out, _total(world * 4).view(world, 4)[rank])
    work = dist.reduce_scatter_tensor(out.zero_(), full, async_op=True)
    work.wait()
    assert torch.equal(out, _total(world * 4).view(world, 4)[rank])
    return True


def test_reduce_scatter_tensor_list_ops_and_async(ranks):
    ranks.run(_reduce_scatter_forms)


def _reduce_scatter_coalesced(rank, world):
    import torch.distributed as dist
    a, b = _values(rank, world * 2), _values(rank, world * 5, torch.float64)
    a_out, b_out = torch.empty(2), torch.empty(5, dtype=torch.float64)
    with dist._coalescing_manager(device=torch.device("cpu"), async_ops=True) as batch:
        dist.reduce_scatter_tensor(a_out, a)
        dist.reduce_scatter_tensor(b_out, b)
    batch.wait()
    assert torch.equal(a_out, _total(world * 2).view(world, 2)[rank])
    assert torch.equal(b_out, _total(world * 5, torch.float64).view(world, 5)[rank])
    return True


def test_coalesced_reduce_scatter_tensor(ranks):
    ranks.run(_reduce_scatter_coalesced)


def _wrong_sizes(rank, world):
    import torch.distributed as dist
    with pytest.raises((ValueError, RuntimeError)):
        dist.all_gather_into_tensor(torch.empty(world * 5 + 1), torch.ones(5))
    with pytest.raises((ValueError, RuntimeError)):
        dist.reduce_scatter_tensor(torch.empty(3), torch.ones(world * 3 + 2))
    with pytest.raises((ValueError, RuntimeError, TypeError)):
        dist.all_gather_into_tensor(torch.empty(world * 5, dtype=torch.float64), torch.ones(5))
    dist.barrier()
    return True


def test_mismatched_sizes_and_dtypes_are_refused_locally(ranks):
    ranks.run(_wrong_sizes)


# ---- what the backend refuses ----------------------------------------------------------------------------
def _refusals(rank, world):
    import torch.distributed as dist
    calls = {
        "all_to_all_single": lambda: dist.all_to_all_single(torch.empty(world), torch.ones(world)),
        "all_to_all": lambda: dist.all_to_all([torch.empty(1) for _ in range(world)],
                                              [torch.ones(1) for _ in range(world)]),
        "reduce": lambda: dist.reduce(torch.ones(2), dst=0),
        "gather": lambda: dist.gather(torch.ones(2), [torch.empty(2) for _ in range(world)] if rank == 0 else None, dst=0),
        "scatter": lambda: dist.scatter(torch.empty(2), [torch.ones(2) for _ in range(world)] if rank == 0 else None, src=0),
    }
    outcome = {}
    for name, call in calls.items():
        try:
            call()
            outcome[name] = "ran"
        except NotImplementedError as exc:
            assert "doesn't support" in str(exc), (name, exc)
            outcome[name] = "refused"
    dist.barrier()                           # nobody is left inside a half-started collective
    return outcome


def test_unsupported_collectives_are_refused_on_every_rank_alike(ranks):
    out = ranks.run(_refusals)
    assert all(o == out[0] for o in out), out
    assert out[0]["all_to_all_single"] == out[0]["all_to_all"] == out[0]["reduce"] == "refused"


def _barrier_and_monitored(rank, world):
    import time
    import torch.distributed as dist
    if rank == 3:
        time.sleep(0.3)
    began = time.monotonic()
    dist.barrier()
    waited = time.monotonic() - began
    work = dist.barrier(async_op=True)
    work.wait()
    return waited


def test_barrier_waits_for_the_slowest_rank(ranks):
    waited = ranks.run(_barrier_and_monitored)
    assert max(waited[:3]) > 0.2 and waited[3] < 0.25


# ---- point to point -----------------------------------------------------------------------------------
def _p2p_same_island_and_across(rank, world):
    import torch.distributed as dist
    dist.barrier()
    across, beside = (rank + 2) % world, rank ^ 1
    for peer, tag in ((across, 11), (beside, 12)):
        out = torch.empty(50)
        ops = [dist.P2POp(dist.isend, _values(rank, 50), peer, tag=tag),
               dist.P2POp(dist.irecv, out, peer, tag=tag)]
        import gpubridge_b200 as gb
        for work in gb.batch_isend_irecv(ops):
            work.wait()
        assert torch.equal(out, _values(peer, 50)), (peer, tag)
    dist.barrier()
    return True


def test_point_to_point_inside_an_island_and_across(ranks):
    ranks.run(_p2p_same_island_and_across)


def _p2p_ring(rank, world):
    import torch.distributed as dist
    dist.barrier()
    right, left = (rank + 1) % world, (rank - 1) % world
    out = torch.empty(8)
    send = dist.isend(_values(rank, 8), right, tag=21)
    recv = dist.irecv(out, left, tag=21)
    send.wait(), recv.wait()
    assert torch.equal(out, _values(left, 8))
    dist.barrier()
    return True


def test_a_ring_of_sends_crosses_both_kinds_of_link(ranks):
    ranks.run(_p2p_ring)


# ---- subgroups ----------------------------------------------------------------------------------------
def _subgroups(rank, world):
    import torch.distributed as dist
    import gpubridge_b200 as gb

    class Seen(gb.CollectiveObserver):
        def __init__(self):
            self.records = []

        def on_collective(self, record):
            self.records.append(record)

    island = dist.new_group([0, 1]), dist.new_group([2, 3])            # every rank creates both
    mixed = dist.new_group([1, 2])
    mine = island[rank // 2]
    seen = Seen()
    gb.add_observer(seen)
    try:
        t = _values(rank, 4)
        dist.all_reduce(t, group=mine)
        want = _values(2 * (rank // 2), 4) + _values(2 * (rank // 2) + 1, 4)
        assert torch.equal(t, want)
        island_record = seen.records[-1]
        if rank in (1, 2):
            t = _values(rank, 4)
            dist.all_reduce(t, group=mixed)
            assert torch.equal(t, _values(1, 4) + _values(2, 4))
            mixed_record = seen.records[-1]
            assert any("bridge" in p.name for p in mixed_record.phases), "two islands: bridged"
        assert not any("bridge" in p.name for p in island_record.phases), "one island: no bridge"
        assert island_record.policy == "native-only"
    finally:
        gb.remove_observer(seen)
    out = torch.empty(2 * 3)
    dist.all_gather_into_tensor(out, _values(rank, 3), group=mine)
    first = 2 * (rank // 2)
    assert torch.equal(out, torch.cat([_values(first, 3), _values(first + 1, 3)]))
    assert dist.get_rank(mine) == rank % 2 and dist.get_world_size(mine) == 2
    dist.barrier()
    for group in (*island, mixed):
        dist.destroy_process_group(group)
    return True


def test_subgroups_inside_an_island_are_native_and_mixed_ones_are_bridged(ranks):
    ranks.run(_subgroups, timeout=120)


def _unsorted_subgroup(rank, world):
    import torch.distributed as dist
    try:
        dist.new_group([2, 0], use_local_synchronization=False)
    except (RuntimeError, ValueError) as exc:
        return "refused" if "ascending" in str(exc) or "sort" in str(exc) else f"other: {exc}"
    return "accepted"


def test_a_subgroup_in_its_own_rank_order_is_sorted_or_refused(ranks):
    out = ranks.run(_unsorted_subgroup, timeout=120)
    assert all(o == out[0] for o in out) and out[0] in ("refused", "accepted"), out


# ---- observers and bookkeeping ----------------------------------------------------------------------------
def _observer_records(rank, world):
    import torch.distributed as dist
    import gpubridge_b200 as gb
    records = []

    class Keep(gb.CollectiveObserver):
        def on_collective(self, record):
            records.append(record)

    watcher = Keep()
    gb.add_observer(watcher)
    try:
        dist.all_reduce(_values(rank, 64))
        dist.broadcast(_values(rank, 8), src=0)
        out = torch.empty(world * 2)
        dist.all_gather_into_tensor(out, _values(rank, 2))
    finally:
        gb.remove_observer(watcher)
    dist.all_reduce(_values(rank, 4))                        # not seen any more
    ops = [r.op for r in records]
    assert ops == ["all_reduce", "broadcast", "all_gather_into_tensor"], ops
    first = records[0]
    assert first.nbytes == 64 * 4 and first.dtype is torch.float32 and first.reduce_op == "sum"
    assert first.policy == "reduce-bridge-broadcast" and records[1].src == 0
    assert [r.seq for r in records] == sorted(r.seq for r in records) and first.ready()
    names = [p.name for p in first.phases]
    assert names and all(gb.elapsed_ms(p.start, p.end) >= 0 for p in first.phases)
    assert gb.in_flight() == []
    return names


def test_observers_see_every_collective_with_its_phases(ranks):
    names = ranks.run(_observer_records)
    assert any("bridge" in n for n in names[0]), names      # a leader crosses the bridge
    assert all(names[r] for r in range(WORLD))


def _topology_facts(rank, world):
    import gpubridge_b200 as gb
    topology = gb.get_topology()
    assert topology.world_size == world and topology.rank == rank
    assert [list(i.ranks) for i in topology.layout.islands] == [[0, 1], [2, 3]]
    assert topology.layout.bridge_ranks == (0, 2)
    assert topology.is_leader == (rank in (0, 2))
    assert topology.island.ranks == ((0, 1) if rank < 2 else (2, 3))
    return topology.policy_name


def test_the_backend_builds_the_same_topology_as_init(ranks):
    assert set(ranks.run(_topology_facts)) == {"reduce-bridge-broadcast"}


def _ddp_with_unused_parameters_and_buffers(rank, world):
    import torch.distributed as dist
    from torch.nn.parallel import DistributedDataParallel as DDP

    class Net(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.used = torch.nn.Linear(4, 4, dtype=torch.float64)
            self.unused = torch.nn.Linear(4, 4, dtype=torch.float64)
            self.register_buffer("steps", torch.zeros(1, dtype=torch.float64))

        def forward(self, x):
            self.steps += 1
            return self.used(x)

    torch.manual_seed(3)
    net = Net()
    with torch.no_grad():
        for p in net.parameters():
            p.copy_(torch.randint(-2, 3, p.shape).double())
    model = DDP(net, find_unused_parameters=True, broadcast_buffers=True)
    x = torch.full((2, 4), float(rank + 1), dtype=torch.float64)
    model(x).sum().backward()
    grads = [p.grad.clone() for p in net.used.parameters()]
    same = [g.clone() for g in grads]
    for g in same:
        dist.all_reduce(g, op=dist.ReduceOp.MAX)
    assert all(torch.equal(a, b) for a, b in zip(grads, same)), "replicas hold different gradients"
    assert net.unused.weight.grad is None or float(net.unused.weight.grad.abs().sum()) == 0.0
    return True


def test_ddp_with_unused_parameters_and_buffers(ranks):
    ranks.run(_ddp_with_unused_parameters_and_buffers, timeout=120)


def _ddp_comm_hook_on_the_backend(rank, world):
    from torch.nn.parallel import DistributedDataParallel as DDP
    import gpubridge_b200 as gb
    torch.manual_seed(0)
    net = torch.nn.Linear(8, 2, dtype=torch.float64)
    with torch.no_grad():
        for p in net.parameters():
            p.copy_(torch.randint(-2, 3, p.shape).double())
    model = DDP(net)
    model.register_comm_hook(None, gb.ddp_comm_hook)
    x = torch.full((4, 8), float(rank), dtype=torch.float64)
    model(x).sum().backward()
    want = sum(torch.full((8,), 4.0 * r, dtype=torch.float64) for r in range(world)) / world
    assert torch.equal(net.weight.grad[0], want)
    return True


def test_the_ddp_hook_works_on_a_backend_group_too(ranks):
    ranks.run(_ddp_comm_hook_on_the_backend, timeout=120)


def _cpu_state_dict_round_trip(rank, world):
    """What a checkpoint needs: object broadcast, a gather of shards, a barrier around it."""
    import torch.distributed as dist
    state = {"weights": _values(rank, 5), "step": 12 + rank}
    shards = [None] * world
    dist.all_gather_object(shards, state)
    dist.barrier()
    assert [s["step"] for s in shards] == [12 + r for r in range(world)]
    assert all(torch.equal(s["weights"], _values(r, 5)) for r, s in enumerate(shards))
    return True


def test_what_checkpointing_needs(ranks):
    ranks.run(_cpu_state_dict_round_trip)
