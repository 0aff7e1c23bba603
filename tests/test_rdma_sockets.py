"""The RDMA-style endpoint over its Unix-domain socket provider: members in different threads
here (each with its own provider and sockets, nothing shared but the names), and - through
``bridge="verbs"`` with ``GPUBRIDGE_VERBS_PROVIDER=sockets`` - in different processes, where it
carries the bridge of every bridged policy against the flat-gloo oracle."""
import threading
import time

import pytest
import torch

from _harness import LAYOUTS, expected_sum, rank_tensor, run_ranks
from gpubridge_b200 import rdma
from gpubridge_b200.ops import _lib

pytestmark = pytest.mark.skipif(not _lib.available(), reason="the native library is not built")


def _members(count, body, leave_together=True, tcp=False, **settings):
    """``body(endpoint, index)`` on ``count`` members.  They close together unless told not to: a
    member that closes is a member that went away, and its peers' endpoints break."""
    names, ready, finished = [None] * count, threading.Barrier(count), threading.Barrier(count)
    out, errors = [None] * count, []

    def run(i):
        endpoint = None
        try:
            def publish(name):
                names[i] = name
                ready.wait(20)
            endpoint = rdma.Endpoint.over_sockets(i, count, publish, lambda: list(names), 20.0,
                                                  tcp_host="127.0.0.1" if tcp else None, **settings)
            out[i] = body(endpoint, i)
            if leave_together:
                finished.wait(30)
        except BaseException as failure:  # noqa: BLE001
            errors.append((i, repr(failure)))
            finished.abort()
        finally:
            if endpoint is not None:
                endpoint.close()

    threads = [threading.Thread(target=run, args=(i,)) for i in range(count)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(60)
    assert not errors, errors
    return out


def test_eager_and_rendezvous_messages_cross_the_sockets():
    small, large = torch.arange(300, dtype=torch.float32), torch.arange(700_000, dtype=torch.float32)

    def body(ep, i):
        deadline = time.monotonic() + 20
        if i == 0:
            ep.wait([ep.send(1, small.data_ptr(), small.nbytes, 5), ep.send(1, large.data_ptr(), large.nbytes, 6)],
                    deadline)
            return ep.telemetry()
        a, b = torch.zeros(300), torch.zeros(700_000)
        ep.wait([ep.recv(0, b.data_ptr(), b.nbytes, 6), ep.recv(0, a.data_ptr(), a.nbytes, 5)], deadline)
        assert torch.equal(a, small) and torch.equal(b, large)
        return ep.telemetry()

    sender, receiver = _members(2, body)
    assert sender["eager_sent"] == 1 and sender["rndv_sent"] == 1 and sender["writes"] >= 2
    assert receiver["mr_misses"] == 1 and not receiver["broken"]


@pytest.mark.parametrize("tcp", [False, True], ids=["unix", "tcp"])
@pytest.mark.parametrize("count", [2, 3, 4])
def test_tagged_collectives_over_sockets(count, tcp):
    def body(ep, i):
        deadline = time.monotonic() + 30
        t = torch.arange(200_000, dtype=torch.float32) + i
        ep.all_reduce(t.data_ptr(), t.numel(), 0, 0, 50_000, 1, deadline)
        b = torch.full((70_000,), float(i))
        ep.broadcast(b.data_ptr(), b.nbytes, count - 1, 1 << 16, 2, deadline)
        return t, b

    want = count * torch.arange(200_000, dtype=torch.float32) + sum(range(count))
    for t, b in _members(count, body, tcp=tcp):
        assert torch.equal(t, want) and torch.equal(b, torch.full((70_000,), float(count - 1)))


def test_a_flood_of_small_messages_respects_the_credits():
    def body(ep, i):
        deadline = time.monotonic() + 30
        payloads = [torch.full((64,), float(k)) for k in range(300)]
        if i == 0:
            ep.wait([ep.send(1, p.data_ptr(), p.nbytes, 9) for p in payloads], deadline)
            return None
        outs = [torch.zeros(64) for _ in range(300)]
        ep.wait([ep.recv(0, o.data_ptr(), o.nbytes, 9) for o in outs], deadline)
        return [float(o[0]) for o in outs]

    out = _members(2, body, data_slots=4, ctrl_slots=3)
    assert out[1] == [float(k) for k in range(300)]


def test_a_member_that_goes_away_breaks_the_others_waits():
    def body(ep, i):
        if i == 1:
            return "left"                                   # closes its endpoint at once
        t = torch.zeros(1 << 20)
        with pytest.raises(RuntimeError):
            ep.wait([ep.recv(1, t.data_ptr(), t.nbytes, 3)], time.monotonic() + 10)
        return ep.telemetry()["broken"]

    assert _members(2, body, leave_together=False) == [True, "left"]


# ---- between processes, as the bridge of the policies ------------------------------------------------
def _through_sockets(rank, topology, policy):
    import gpubridge_b200 as gb
    assert topology.peers[rank].bridge == "verbs"
    world = topology.world_size
    for n in (1, 1000, 300_001):
        for dtype in (torch.float32, torch.int64):
            t = rank_tensor(rank, n, dtype)
            gb.all_reduce(t)
            assert torch.equal(t, expected_sum(world, n, dtype)), (n, dtype)
    t = rank_tensor(rank, 5000)
    gb.broadcast(t, 3)
    assert torch.equal(t, rank_tensor(3, 5000))
    return topology.policy_name


@pytest.mark.parametrize("policy, provider", [("auto", "sockets"), ("pipelined-reduce-bridge-broadcast", "sockets"),
                                              ("sharded-bridge", "sockets"), ("auto", "tcp")])
def test_policies_over_the_verbs_bridge_between_processes(tmp_path, policy, provider):
    out = run_ranks(LAYOUTS["2+2"], _through_sockets, tmp_path, policy,
                    init={"bridge": "verbs", "policy": policy},
                    env={"GPUBRIDGE_VERBS_PROVIDER": provider}, timeout=120)
    assert len(set(out)) == 1


def test_without_a_provider_the_name_still_refuses(tmp_path):
    run_ranks(LAYOUTS["2+2"], _through_sockets, tmp_path, "auto", init={"bridge": "verbs"},
              expect_error="provider", timeout=60)
