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
