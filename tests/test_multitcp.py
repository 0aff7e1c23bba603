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


def _native_equals_python(members: int):
    """The collectives inside the library against the same algorithms in Python, thread per
    member, every dtype and op, sizes around the chunk boundaries: bit for bit."""
    import threading
    import time
    from datetime import timedelta
    from gpubridge_b200.multitcp import MultiTcpTransport, Worker

    def link():
        workers = [Worker(i, members, 2, "127.0.0.1") for i in range(members)]
        addresses = [w.address() for w in workers]
        threads = [threading.Thread(target=w.connect, args=(addresses, 20.0)) for w in workers]
        [t.start() for t in threads]
        [t.join() for t in threads]
        return [MultiTcpTransport(w, list(range(members)), i, timedelta(seconds=30), 4096)
                for i, w in enumerate(workers)]

    def values(rank, n, dtype):
        g = torch.Generator().manual_seed(100 * rank + n)
        if dtype.is_floating_point:
            t = (torch.randn(n, generator=g) * 3).to(dtype)
            if n > 4:
                t[3] = float("nan") if rank == 0 else 1.0
            return t
        return torch.randint(-100, 100, (n,), generator=g).to(dtype)

    def run(transports, fn):
        errors = []

        def one(tr, rank):
            try:
                fn(tr, rank)
            except BaseException as exc:  # noqa: BLE001
                errors.append(exc)
        threads = [threading.Thread(target=one, args=(tr, r)) for r, tr in enumerate(transports)]
        [t.start() for t in threads]
        [t.join() for t in threads]
        assert not errors, errors

    import os
    results = {}
    for native in ("1", "0"):
        os.environ["GPUBRIDGE_TAGGED_NATIVE"] = native
        transports = link()
        got = {}

        def work(tr, rank, got=got):
            for dtype in (torch.float32, torch.bfloat16, torch.float16, torch.float64,
                          torch.int8, torch.uint8, torch.int32, torch.int64):
                for n in (1, 2, 1023, 1024, 1025, 5000):
                    for op in ("sum", "max", "min"):
                        t = values(rank, n, dtype)
                        tr.all_reduce(t, op)
                        got[(rank, str(dtype), n, op)] = t.clone()
            t = values(rank, 3000, torch.float32)
            tr.broadcast(t, members - 1)
            got[(rank, "bcast")] = t.clone()
        try:
            run(transports, work)
        finally:
            for tr in transports:
                tr.close()
        results[native] = got
    os.environ.pop("GPUBRIDGE_TAGGED_NATIVE", None)
    assert results["1"].keys() == results["0"].keys()
    for key, want in results["0"].items():
        have = results["1"][key]
        same = torch.equal(have.view(torch.uint8), want.view(torch.uint8)) if have.dtype != torch.bool else True
        if not same:                      # NaN payload bits may differ; values must not
            assert torch.equal(have.isnan(), want.isnan()), key
            assert torch.equal(have.nan_to_num(), want.nan_to_num()), key
    assert torch.equal(results["1"][(0, "bcast")], values(members - 1, 3000, torch.float32))


def test_native_collectives_equal_python_two_members():
    _native_equals_python(2)


def test_native_collectives_equal_python_ring():
    _native_equals_python(3)
