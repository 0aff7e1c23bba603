"""The native multi-stream TCP bridge: every bridged policy against the flat-gloo oracle, and
a worker whose peer goes away (reference: tests/test_multitcp.py)."""
import pytest
import torch

from _harness import LAYOUTS, expected_sum, rank_tensor, run_ranks


def _through_tcp(rank, topology):
    import gpubridge_b200 as gb
    assert topology.peers[rank].bridge == "multitcp"
    world = topology.world_size
    for dtype in (torch.float32, torch.int64, torch.bfloat16):
        for n in (1, 1031, 300_000):
            t = rank_tensor(rank, n, dtype)
            gb.all_reduce(t)
            assert torch.equal(t, expected_sum(world, n, dtype)), (dtype, n)
    t = rank_tensor(rank, 50)
    gb.all_reduce(t, gb.ReduceOp.MAX)
    assert torch.equal(t, rank_tensor(world - 1, 50))
    t = rank_tensor(rank, 2000)
    gb.broadcast(t, world - 1)
    assert torch.equal(t, rank_tensor(world - 1, 2000))
    out = torch.empty(world * 10)
    gb.all_gather_into_tensor(out, rank_tensor(rank, 10))
    assert torch.equal(out, torch.cat([rank_tensor(r, 10) for r in range(world)]))
    return True


@pytest.mark.parametrize("policy", ["auto", "pipelined-reduce-bridge-broadcast", "sharded-bridge"])
def test_policies_over_multitcp(tmp_path, policy):
    run_ranks(LAYOUTS["2+2"], _through_tcp, tmp_path, init={"bridge": "multitcp", "policy": policy},
              env={"GPUBRIDGE_MULTITCP_CHUNK_BYTES": "64K", "GPUBRIDGE_CHUNK_BYTES": "32K"})


def test_three_islands_ring(tmp_path):
    run_ranks(("nvidia",) * 3, _through_tcp, tmp_path, init={"bridge": "multitcp"},
              env={"GPUBRIDGE_ISLANDS": "1,1,1", "GPUBRIDGE_MULTITCP_STREAMS": "2"})


def test_worker_reports_a_vanished_peer():
    import threading
    import time
    from gpubridge_b200.multitcp import Worker
    a, b = Worker(0, 2, 2, "127.0.0.1"), Worker(1, 2, 2, "127.0.0.1")
    addresses = [a.address(), b.address()]
    t = threading.Thread(target=b.connect, args=(addresses, 10.0))
    t.start()
    a.connect(addresses, 10.0)
    t.join()
    buf = torch.zeros(4, dtype=torch.int64)
    src = torch.arange(4)
    r = a.recv(1, buf.data_ptr(), 32, 7)
    s = b.send(0, src.data_ptr(), 32, 7)
    b.wait([s], time.monotonic() + 5)
    a.wait([r], time.monotonic() + 5)
    assert torch.equal(buf, src)
    pending = a.recv(1, buf.data_ptr(), 32, 8)
    b.close()                                       # the peer goes away
    with pytest.raises(RuntimeError, match="multitcp"):
        a.wait([pending], time.monotonic() + 5)
    with pytest.raises(RuntimeError):
        a.send(1, src.data_ptr(), 32, 9)            # the worker stays broken
    a.close()


def _expected(inputs, op):
    """What the native collectives must produce, bit for bit, rebuilt from the two rules
    gpubridge_b200.tagged documents: two members fold the peer's values into their own; a ring
    folds segment j starting at member j and walking upward."""
    from gpubridge_b200.tagged import ring_order, segments
    fold = {"sum": torch.add, "max": torch.maximum, "min": torch.minimum}[op]
    members = len(inputs)
    if members == 2:
        return [fold(inputs[0], inputs[1]), fold(inputs[1], inputs[0])]
    out = torch.empty_like(inputs[0])
    for j, (start, length) in enumerate(segments(out.numel(), members)):
        order = ring_order(j, members)
        acc = inputs[order[0]][start:start + length].clone()
        for member in order[1:]:
            acc = fold(inputs[member][start:start + length], acc)      # own value first, as the worker folds
        out[start:start + length] = acc
    return [out] * members


def _native_matches_the_documented_order(members: int):
    """The collectives inside the library, a thread per member, every dtype and op, sizes
    around the chunk boundaries, against :func:`_expected`."""
    import threading
    from datetime import timedelta
    from gpubridge_b200.multitcp import MultiTcpTransport, Worker

    workers = [Worker(i, members, 2, "127.0.0.1") for i in range(members)]
    addresses = [w.address() for w in workers]
    joiners = [threading.Thread(target=w.connect, args=(addresses, 20.0)) for w in workers]
    [t.start() for t in joiners]
    [t.join() for t in joiners]
    transports = [MultiTcpTransport(w, list(range(members)), i, timedelta(seconds=30), 4096)
                  for i, w in enumerate(workers)]

    def values(rank, n, dtype):
        g = torch.Generator().manual_seed(100 * rank + n)
        if dtype.is_floating_point:
            t = (torch.randn(n, generator=g) * 3).to(dtype)
            if n > 4:
                t[3] = float("nan") if rank == 0 else 1.0
            return t
        return torch.randint(-100, 100, (n,), generator=g).to(dtype)

    cases = [(dtype, n, op)
             for dtype in (torch.float32, torch.bfloat16, torch.float16, torch.float64,
                           torch.int8, torch.uint8, torch.int32, torch.int64)
             for n in (1, 2, 1023, 1024, 1025, 5000) for op in ("sum", "max", "min")]
    got, errors = {}, []

    def member(rank):
        try:
            transports[rank].prove(__import__("time").monotonic() + 20)
            for dtype, n, op in cases:
                t = values(rank, n, dtype)
                transports[rank].all_reduce(t, op)
                got[(rank, dtype, n, op)] = t
            t = values(rank, 3000, torch.float32)
            transports[rank].broadcast(t, members - 1)
            got[(rank, "bcast")] = t
        except BaseException as exc:  # noqa: BLE001
            errors.append(exc)

    threads = [threading.Thread(target=member, args=(r,)) for r in range(members)]
    try:
        [t.start() for t in threads]
        [t.join() for t in threads]
    finally:
        for tr in transports:
            tr.close()
    assert not errors, errors
    for dtype, n, op in cases:
        want = _expected([values(r, n, dtype) for r in range(members)], op)
        for rank in range(members):
            have = got[(rank, dtype, n, op)]
            if not torch.equal(have.view(torch.uint8), want[rank].view(torch.uint8)):
                # NaN payload bits may differ between the library and torch; values must not
                assert torch.equal(have.isnan(), want[rank].isnan()), (dtype, n, op, rank)
                assert torch.equal(have.nan_to_num(), want[rank].nan_to_num()), (dtype, n, op, rank)
    for rank in range(members):
        assert torch.equal(got[(rank, "bcast")], values(members - 1, 3000, torch.float32))


def test_native_collectives_two_members():
    _native_matches_the_documented_order(2)


def test_native_collectives_ring():
    _native_matches_the_documented_order(3)


def test_native_collectives_ring_of_five():
    _native_matches_the_documented_order(5)


def _p2p_beside_a_tagged_bridge(rank, world):
    import torch.distributed as dist
    from gpubridge_b200.p2p import GlooLink
    dist.barrier()
    peer = {0: 2, 2: 0}.get(rank)
    if peer is not None:
        data = torch.arange(70_001, dtype=torch.float32)
        if rank == 0:
            dist.send(data, peer, tag=4)
        else:
            got = torch.zeros(70_001)
            dist.recv(got, peer, tag=4)
            assert torch.equal(got, data)
        assert isinstance(dist.distributed_c10d._get_default_group()._engine.link, GlooLink)
    t = torch.ones(100) * rank
    dist.all_reduce(t)
    assert float(t[0]) == 6.0
    dist.barrier()
    return True


def test_cross_island_point_to_point_with_the_multitcp_bridge(tmp_path):
    """A bridge that brings no point-to-point wire of its own leaves that traffic to the job's
    Gloo group instead of refusing it."""
    from _harness import TWO_BY_TWO, run_ranks
    run_ranks(TWO_BY_TWO, _p2p_beside_a_tagged_bridge, tmp_path, mode="backend", timeout=120,
              env={"GPUBRIDGE_BRIDGE": "multitcp"})
