"""The native multi-stream TCP worker (``csrc/gb_tcp.cpp``) member by member, in threads of this
process: its settings, messages matched by (peer, tag) whatever order they are posted in, one
message per tag in order, sizes from nothing to many chunks over one and many connections per
peer, a size mismatch as an error, what was sent before a close still arriving, a member that
never connects, a deadline on a message nobody sends, close with operations outstanding, bad
arguments; and, as ranks, settings that differ between leaders.
(Reference: tests/test_multitcp.py and the unit tests of its multitcp crate.)"""
import threading
import time

import pytest
import torch

from _harness import LAYOUTS, per_rank, run_ranks
from gpubridge_b200.ops import _lib

pytestmark = pytest.mark.skipif(not _lib.available(), reason="the native library is not built")


def connected(count, streams=2):
    from gpubridge_b200.multitcp import Worker
    workers = [Worker(i, count, streams, "127.0.0.1") for i in range(count)]
    addresses = [w.address() for w in workers]
    threads = [threading.Thread(target=w.connect, args=(addresses, 20.0)) for w in workers]
    for t in threads:
        t.start()
    for t in threads:
        t.join(30)
    return workers


def close_all(workers):
    threads = [threading.Thread(target=w.close) for w in workers]
    for t in threads:
        t.start()
    for t in threads:
        t.join(20)


def soon(seconds=10.0):
    return time.monotonic() + seconds


# ---- settings ---------------------------------------------------------------------------------------------
def test_settings(monkeypatch):
    from gpubridge_b200 import multitcp
    monkeypatch.delenv(multitcp.STREAMS_ENV, raising=False)
    assert multitcp.streams_setting() == 4
    monkeypatch.setenv(multitcp.STREAMS_ENV, "16")
    assert multitcp.streams_setting() == 16
    for bad in ("0", "65", "-1"):
        monkeypatch.setenv(multitcp.STREAMS_ENV, bad)
        with pytest.raises(ValueError, match="between 1 and 64"):
            multitcp.streams_setting()
    monkeypatch.setenv(multitcp.STREAMS_ENV, "many")
    with pytest.raises(ValueError):
        multitcp.streams_setting()


def test_the_listening_address_follows_the_interface_settings(monkeypatch):
    import socket
    from types import SimpleNamespace as Address

    import psutil

    from gpubridge_b200 import multitcp
    monkeypatch.delenv(multitcp.IFADDR_ENV, raising=False)
    monkeypatch.delenv(multitcp.IFNAME_ENV, raising=False)
    assert multitcp.listen_address() == "127.0.0.1"
    table = {"ib0": [Address(family=socket.AF_INET6, address="fe80::1"), Address(family=socket.AF_INET, address="10.9.8.7")],
             "v6only": [Address(family=socket.AF_INET6, address="fe80::2")]}
    monkeypatch.setattr(psutil, "net_if_addrs", lambda: table)
    monkeypatch.setenv(multitcp.IFNAME_ENV, "ib0")
    assert multitcp.listen_address() == "10.9.8.7"
    for missing in ("eth9", "v6only"):
        monkeypatch.setenv(multitcp.IFNAME_ENV, missing)
        with pytest.raises(ValueError, match="no such interface with an IPv4 address"):
            multitcp.listen_address()
    monkeypatch.setenv(multitcp.IFADDR_ENV, "192.168.1.5")          # an explicit address wins over a name
    assert multitcp.listen_address() == "192.168.1.5"


def test_a_worker_that_cannot_listen_says_why():
    from gpubridge_b200.multitcp import Worker
    with pytest.raises(RuntimeError, match="multitcp"):
        Worker(0, 2, 2, "203.0.113.77")                            # not an address of this machine
    with pytest.raises(RuntimeError, match="multitcp"):
        Worker(0, 2, 2, "not-an-address")


# ---- messages ----------------------------------------------------------------------------------------------
@pytest.mark.parametrize("streams", [1, 2, 8])
def test_sizes_from_nothing_to_many_megabytes(streams):
    a, b = connected(2, streams)
    try:
        for n in (0, 1, 7, 4096, 1_000_003, 6_000_000):
            data = (torch.arange(n, dtype=torch.int64) * 7 + 1).to(torch.int32)
            room = torch.zeros(n, dtype=torch.int32)
            r = b.recv(0, room.data_ptr(), room.nbytes, 5)
            s = a.send(1, data.data_ptr(), data.nbytes, 5)
            a.wait([s], soon(30))
            b.wait([r], soon(30))
            assert torch.equal(room, data), n
    finally:
        close_all([a, b])


def test_receives_are_matched_by_peer_and_tag_in_any_order():
    workers = connected(3)
    try:
        payloads = {(src, tag): torch.full((1000,), float(10 * src + tag)) for src in (1, 2) for tag in (1, 2, 3)}
        rooms = {key: torch.zeros(1000) for key in payloads}
        # member 0 posts its receives in one order, the others send in another
        receives = [workers[0].recv(src, rooms[(src, tag)].data_ptr(), 4000, tag)
                    for tag in (3, 1, 2) for src in (2, 1)]
        sends = {1: [], 2: []}
        for src in (1, 2):
            for tag in (1, 2, 3):
                sends[src].append(workers[src].send(0, payloads[(src, tag)].data_ptr(), 4000, tag))
        for src in (1, 2):
            workers[src].wait(sends[src], soon())
        workers[0].wait(receives, soon())
        for key, room in rooms.items():
            assert torch.equal(room, payloads[key]), key
    finally:
        close_all(workers)


def test_messages_on_one_tag_arrive_in_the_order_sent_and_may_come_early():
    a, b = connected(2, streams=4)
    try:
        payloads = [torch.full((5000,), float(k)) for k in range(12)]
        sends = [a.send(1, p.data_ptr(), p.nbytes, 9) for p in payloads]        # nothing is posted on the other side yet
        time.sleep(0.2)
        rooms = [torch.zeros(5000) for _ in range(12)]
        receives = [b.recv(0, r.data_ptr(), r.nbytes, 9) for r in rooms]
        b.wait(receives, soon())
        a.wait(sends, soon())
        assert [float(r[0]) for r in rooms] == [float(k) for k in range(12)]
    finally:
        close_all([a, b])


def test_a_message_of_the_wrong_size_is_an_error_not_garbage():
    a, b = connected(2)
    try:
        data, room = torch.ones(100), torch.zeros(50)
        s = a.send(1, data.data_ptr(), data.nbytes, 3)
        r = b.recv(0, room.data_ptr(), room.nbytes, 3)
        with pytest.raises(RuntimeError, match="400|200|size|length"):
            b.wait([r], soon(5))
        with pytest.raises(RuntimeError):                          # the worker stays broken
            b.recv(0, room.data_ptr(), room.nbytes, 4)
        try:
            a.wait([s], soon(2))
        except RuntimeError:
            pass                                                   # the peer went away under it: either is fine
    finally:
        close_all([a, b])


def test_what_was_sent_before_a_close_still_arrives():
    a, b = connected(2)
    data, room = torch.arange(70_000, dtype=torch.float32), torch.zeros(70_000)
    s = a.send(1, data.data_ptr(), data.nbytes, 1)
    a.wait([s], soon())
    a.close()                                                      # the sender is gone before anybody asks
    try:
        r = b.recv(0, room.data_ptr(), room.nbytes, 1)
        b.wait([r], soon())
        assert torch.equal(room, data)
    finally:
        b.close()


def test_a_message_nobody_sends_trips_the_deadline_and_breaks_the_worker():
    a, b = connected(2)
    try:
        room = torch.zeros(10)
        started = time.monotonic()
        with pytest.raises(RuntimeError, match="multitcp"):
            b.wait([b.recv(0, room.data_ptr(), room.nbytes, 1)], soon(0.4))
        assert time.monotonic() - started < 5
        with pytest.raises(RuntimeError):
            b.all_reduce(room.data_ptr(), 10, 0, 0, 10, 1, soon(1))
    finally:
        close_all([a, b])


def test_a_member_that_never_connects_trips_connects_own_limit():
    from gpubridge_b200.multitcp import Worker
    a, b = Worker(0, 2, 2, "127.0.0.1"), Worker(1, 2, 2, "127.0.0.1")
    try:
        started = time.monotonic()
        with pytest.raises(RuntimeError, match="multitcp"):
            b.connect([a.address(), b.address()], 0.5)             # member 0 listens but never dials back / accepts
        assert time.monotonic() - started < 10
    finally:
        a.close()
        b.close()


def test_close_with_operations_outstanding_returns_and_leaves_memory_alone():
    a, b = connected(2)
    room = torch.full((1 << 18,), 7.0)
    a.recv(1, room.data_ptr(), room.nbytes, 4)                     # never matched, never waited for
    big = torch.ones(1 << 22)
    b.send(0, big.data_ptr(), big.nbytes, 99)                      # nobody receives tag 99
    started = time.monotonic()
    close_all([a, b])
    assert time.monotonic() - started < 15
    assert torch.equal(room, torch.full((1 << 18,), 7.0))          # nothing wrote into it afterwards
    with pytest.raises(Exception):
        a.send(1, big.data_ptr(), 8, 1)                            # a closed worker refuses instead of crashing


def test_bad_arguments_are_refused():
    a, b = connected(2)
    try:
        t = torch.zeros(4)
        for peer in (-1, 2, 0):                                    # out of range, and itself
            with pytest.raises(RuntimeError, match="multitcp"):
                a.send(peer, t.data_ptr(), t.nbytes, 1)
        with pytest.raises(RuntimeError, match="multitcp"):
            a.all_reduce(t.data_ptr(), 4, 99, 0, 4, 1, soon(1))    # no such element type
    finally:
        close_all([a, b])


# ---- as the bridge: what leaders must agree on ----------------------------------------------------------------
@pytest.mark.parametrize("what, envs, message", [
    ("a bad stream count on one leader", {2: {"GPUBRIDGE_MULTITCP_STREAMS": "0"}}, "between 1 and 64"),
    ("a bad chunk size on one leader", {0: {"GPUBRIDGE_MULTITCP_CHUNK_BYTES": "13"}}, "multiple of 8"),
    ("an interface that is not there", {0: {"GPUBRIDGE_MULTITCP_IFNAME": "nosuch0"}}, "no such interface"),
    ("another stream count on one leader", {2: {"GPUBRIDGE_MULTITCP_STREAMS": "7"}}, "GPUBRIDGE_MULTITCP_STREAMS differs"),
    ("another chunk size on one leader", {0: {"GPUBRIDGE_MULTITCP_CHUNK_BYTES": "64K"}}, "GPUBRIDGE_MULTITCP_CHUNK_BYTES differs"),
])
def test_one_leaders_trouble_fails_init_on_every_rank(tmp_path, what, envs, message):
    errors = run_ranks(LAYOUTS["2+2"], per_rank, tmp_path, envs, {"bridge": "multitcp"}, mode="plain",
                       expect_error=message, timeout=90)
    assert len(errors) == 4 and all("could not be set up" in e for e in errors)


def test_close_from_another_thread_ends_a_blocked_wait_before_the_worker_is_freed():
    a, b = connected(2)
    room = torch.zeros(64)
    seen = {}

    def waits():
        try:
            a.wait([a.recv(1, room.data_ptr(), room.nbytes, 3)], soon(30))
            seen["wait"] = "returned"
        except RuntimeError as failure:
            seen["wait"] = str(failure)

    thread = threading.Thread(target=waits)
    thread.start()
    time.sleep(0.3)
    started = time.monotonic()
    a.close()
    thread.join(10)
    assert not thread.is_alive() and time.monotonic() - started < 8
    assert seen["wait"].startswith("multitcp")
    with pytest.raises(RuntimeError, match="closed"):
        a.address()
    a.abort()
    a.close()
    b.close()
