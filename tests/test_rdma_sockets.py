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


# ---- settings of the verbs bridge ---------------------------------------------------------------------
def test_endpoint_settings_parse_and_refuse_bad_values(monkeypatch):
    from gpubridge_b200 import rdma_transport
    for name in rdma_transport.ENDPOINT_SETTINGS:
        monkeypatch.delenv(name, raising=False)
    assert rdma_transport.endpoint_settings() == {"eager_max": 16 << 10, "data_slots": 16, "max_write": 1 << 20,
                                                  "unexpected_max": 64 << 20, "mr_cache": 64}
    monkeypatch.setenv("GPUBRIDGE_VERBS_SLOT_BYTES", "64K")
    monkeypatch.setenv("GPUBRIDGE_VERBS_CREDITS", "4")
    told = rdma_transport.endpoint_settings()
    assert told["eager_max"] == 65536 and told["data_slots"] == 4
    monkeypatch.setenv("GPUBRIDGE_VERBS_SLOT_BYTES", "1001")
    with pytest.raises(ValueError, match="GPUBRIDGE_VERBS_SLOT_BYTES.*multiple of 8"):
        rdma_transport.endpoint_settings()
    monkeypatch.setenv("GPUBRIDGE_VERBS_SLOT_BYTES", "64K")
    monkeypatch.setenv("GPUBRIDGE_VERBS_GPU_PATH", "staged")
    router = rdma_transport.Router(device_registration=True)
    from types import SimpleNamespace
    device_tensor = SimpleNamespace(device=SimpleNamespace(type="cuda", index=0), nbytes=1 << 20,
                                    is_contiguous=lambda: True, data_ptr=lambda: 0x1000)
    route = router.route(device_tensor)
    assert route.how == "bounce" and "GPUBRIDGE_VERBS_GPU_PATH=staged" in route.why
    monkeypatch.setenv("GPUBRIDGE_VERBS_GPU_PATH", "sideways")
    with pytest.raises(ValueError, match="GPUBRIDGE_VERBS_GPU_PATH"):
        rdma_transport.Router()


def _observed(rank, topology, out_dir):
    import gpubridge_b200 as gb
    t = rank_tensor(rank, 70_001)
    gb.all_reduce(t)
    assert torch.equal(t, expected_sum(topology.world_size, 70_001))
    gb.broadcast(t, 0)
    told = None if topology.bridge is None else topology.bridge.describe()["endpoint"]
    return told


def test_the_bridge_honours_its_settings_and_writes_its_observations(tmp_path):
    import json
    out = run_ranks(LAYOUTS["2+2"], _observed, tmp_path, str(tmp_path), init={"bridge": "verbs"}, timeout=120,
                    env={"GPUBRIDGE_VERBS_PROVIDER": "sockets", "GPUBRIDGE_VERBS_SLOT_BYTES": "1K",
                         "GPUBRIDGE_VERBS_CREDITS": "2", "GPUBRIDGE_VERBS_WRITE_BYTES": "8K",
                         "GPUBRIDGE_VERBS_OBSERVE": str(tmp_path / "observed-%r.jsonl"), "GPUBRIDGE_JOB_ID": "job-77"})
    leaders = [told for told in out if told is not None]
    assert len(leaders) == 2
    # 280 KB above a 1 KB slot: everything went by rendezvous, in writes of 8 KB
    assert all(told["rndv_sent"] >= 1 and told["writes"] >= 280_004 // 8192 for told in leaders)
    files = sorted(tmp_path.glob("observed-*.jsonl"))
    assert [f.name for f in files] == ["observed-0.jsonl", "observed-2.jsonl"]          # the leaders' files, finished
    records = [json.loads(line) for line in files[0].read_text().splitlines()]
    calls = [r for r in records if r["kind"] == "bridge_call"]
    assert len(calls) == 2 and all(r["job"] == "job-77" and r["bridge"] == "verbs" and r["route"] == "plain" for r in calls)
    assert any(r["nbytes"] == 280_004 and r["ms"] > 0 for r in calls)
    assert [r["kind"] for r in records][-2:] == ["endpoint", "closed"]
    assert not any("rkey" in json.dumps(r) or "key" in " ".join(r) for r in records)


@pytest.mark.parametrize("envs, message", [
    ({2: {"GPUBRIDGE_VERBS_SLOT_BYTES": "2K"}}, "verbs settings differ"),
    ({0: {"GPUBRIDGE_VERBS_CREDITS": "0"}}, "GPUBRIDGE_VERBS_CREDITS"),
])
def test_leaders_whose_settings_differ_or_are_bad_fail_init_on_every_rank(tmp_path, envs, message):
    from _harness import per_rank
    common = {"GPUBRIDGE_VERBS_PROVIDER": "sockets"}
    per = {r: dict(common, **envs.get(r, {})) for r in range(4)}
    errors = run_ranks(LAYOUTS["2+2"], per_rank, tmp_path, per, {"bridge": "verbs"}, mode="plain",
                       expect_error=message, timeout=90)
    assert len(errors) == 4 and all("could not be set up" in e for e in errors)
