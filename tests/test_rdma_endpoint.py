"""The RDMA-style endpoint (csrc/gb_rdma.cpp) over its in-process fabric: eager and rendezvous
messages, ordering and tag matching, messages that arrive early, flow control that never lets a
send find its receiver unprepared, the registration cache, what telemetry reports - and the
failure rule under injected faults: an errored, dropped, corrupted or refused operation and a
member that dies put the endpoint into a broken state that fails everything with the first
reason, in bounded time.  Collectives ride on it through the shared tagged algorithms.
(The reference tests its verbs endpoint the same way, on a mock fabric inside one process:
src/gpubridge/verbs/crate/src/mock.rs.)"""
import threading
import time

import pytest
import torch

from gpubridge_b200 import rdma
from gpubridge_b200.ops import _lib

pytestmark = pytest.mark.skipif(not _lib.available(), reason="the native library is not built")


@pytest.fixture()
def fabric():
    made = []

    def build(members=2, **settings):
        f = rdma.MockFabric(members)
        made.append(f)
        return f, [f.endpoint(i, **settings) for i in range(members)]

    yield build
    for f in made:
        f.close()


def soon(seconds=5.0):
    return time.monotonic() + seconds


def exchange(a, b, data, tag=1, receive_first=True):
    out = torch.zeros_like(data)
    if receive_first:
        r = b.recv(a.index, out.data_ptr(), out.nbytes, tag)
        s = a.send(b.index, data.data_ptr(), data.nbytes, tag)
    else:
        s = a.send(b.index, data.data_ptr(), data.nbytes, tag)
        time.sleep(0.05)
        r = b.recv(a.index, out.data_ptr(), out.nbytes, tag)
    a.wait([s], soon())
    b.wait([r], soon())
    return out


@pytest.mark.parametrize("n", [0, 1, 4096, 4097, 300_000])
@pytest.mark.parametrize("receive_first", [True, False])
def test_messages_of_every_size_arrive_whole(fabric, n, receive_first):
    f, (a, b) = fabric(eager_max=16384)
    data = (torch.arange(n) % 251).to(torch.float32)
    assert torch.equal(exchange(a, b, data, receive_first=receive_first), data)
    counters = a.telemetry()
    assert counters["eager_sent"] + counters["rndv_sent"] == 1
    assert (counters["rndv_sent"] == 1) == (data.nbytes > 16384)
    assert f.stats()["rnr"] == 0, "a send found no receive posted: flow control failed"


def test_large_messages_are_written_in_place_in_pieces(fabric):
    f, (a, b) = fabric(eager_max=1024, max_write=10_000)
    data = torch.arange(100_000, dtype=torch.int64)                   # 800 000 bytes: 80 writes
    assert torch.equal(exchange(a, b, data), data)
    assert f.stats()["writes"] == 80 and a.telemetry()["writes"] == 80
    assert b.telemetry()["rndv_recv"] == 1 and b.telemetry()["bytes_recv"] == data.nbytes


def test_one_tag_keeps_order_and_tags_do_not_mix(fabric):
    f, (a, b) = fabric()
    outs = [torch.zeros(8) for _ in range(30)]
    recvs = [b.recv(0, o.data_ptr(), o.nbytes, 7) for o in outs]
    payloads = [torch.full((8,), float(i)) for i in range(30)] + [torch.full((8,), 99.0)]   # kept alive
    sends = [a.send(1, payloads[i].data_ptr(), 32, 7) for i in range(30)]
    other = torch.zeros(8)
    r9 = b.recv(0, other.data_ptr(), 32, 9)
    s9 = a.send(1, payloads[30].data_ptr(), 32, 9)
    a.wait(sends + [s9], soon())
    b.wait(recvs + [r9], soon())
    assert [float(o[0]) for o in outs] == [float(i) for i in range(30)] and float(other[0]) == 99.0


def test_early_messages_wait_for_their_receives_in_any_tag_order(fabric):
    f, (a, b) = fabric(eager_max=1024)
    small, large = torch.full((16,), 3.0), torch.arange(5000, dtype=torch.float32)
    s1 = a.send(1, small.data_ptr(), small.nbytes, 21)
    s2 = a.send(1, large.data_ptr(), large.nbytes, 22)
    time.sleep(0.1)
    assert b.telemetry()["unexpected"] == 2
    got_large, got_small = torch.zeros(5000), torch.zeros(16)
    r2 = b.recv(0, got_large.data_ptr(), got_large.nbytes, 22)        # the later message first
    r1 = b.recv(0, got_small.data_ptr(), got_small.nbytes, 21)
    b.wait([r1, r2], soon())
    a.wait([s1, s2], soon())
    assert torch.equal(got_small, small) and torch.equal(got_large, large)
    assert b.telemetry()["unexpected_bytes_now"] == 0


def test_credits_hold_back_a_flood_and_every_message_still_arrives(fabric):
    f, (a, b) = fabric(data_slots=4, ctrl_slots=3)
    # the first credit message back to the sender is late, so the sender is certain to run dry
    f.inject("delay", src=1, dst=0, on="send", nth=1, milliseconds=200)
    payloads = [torch.full((64,), float(i)) for i in range(200)]
    sends = [a.send(1, p.data_ptr(), p.nbytes, 1) for p in payloads]  # far more than four slots
    outs = [torch.zeros(64) for _ in range(200)]
    recvs = [b.recv(0, o.data_ptr(), o.nbytes, 1) for o in outs]
    a.wait(sends, soon(10))
    b.wait(recvs, soon(10))
    assert [float(o[0]) for o in outs] == [float(i) for i in range(200)]
    assert f.stats()["rnr"] == 0
    assert a.telemetry()["credit_stalls"] > 0 and b.telemetry()["credit_msgs"] > 0


def test_two_members_flooding_each_other_do_not_lock_up(fabric):
    f, (a, b) = fabric(data_slots=2, ctrl_slots=2, eager_max=256)
    big = torch.arange(2000, dtype=torch.float32)                      # rendezvous both ways, with eager in between
    results = {}

    def run(me, peer, name):
        sends, recvs, outs = [], [], []
        for i in range(40):
            outs.append(torch.zeros(2000) if i % 4 == 0 else torch.zeros(32))
            recvs.append(me.recv(peer, outs[-1].data_ptr(), outs[-1].nbytes, i))
            payload = big if i % 4 == 0 else torch.full((32,), float(i))
            results.setdefault(name + "keep", []).append(payload)
            sends.append(me.send(peer, payload.data_ptr(), payload.nbytes, i))
        me.wait(sends + recvs, soon(20))
        results[name] = outs

    threads = [threading.Thread(target=run, args=(a, 1, "a")), threading.Thread(target=run, args=(b, 0, "b"))]
    [t.start() for t in threads]
    [t.join(30) for t in threads]
    assert "a" in results and "b" in results, (a.telemetry(), b.telemetry())
    assert all(torch.equal(results["a"][i], big) for i in range(0, 40, 4))
    assert all(float(results["b"][i][0]) == float(i) for i in range(40) if i % 4)
    assert f.stats()["rnr"] == 0


def test_registrations_are_cached_evicted_and_invalidated(fabric):
    f, (a, b) = fabric(eager_max=64, mr_cache=2)
    buffers = [torch.zeros(1000) for _ in range(3)]
    data = torch.arange(1000, dtype=torch.float32)

    def into(buffer):
        r = b.recv(0, buffer.data_ptr(), buffer.nbytes, 1)
        s = a.send(1, data.data_ptr(), data.nbytes, 1)
        a.wait([s], soon()), b.wait([r], soon())

    into(buffers[0]); into(buffers[0]); into(buffers[0])
    t = b.telemetry()
    assert (t["mr_misses"], t["mr_hits"]) == (1, 2)
    into(buffers[1]); into(buffers[2])                                  # a third registration evicts the oldest
    t = b.telemetry()
    assert t["mr_misses"] == 3 and t["mr_evictions"] == 1 and t["mr_entries"] == 2
    into(buffers[0])                                                   # evicted: registered again
    assert b.telemetry()["mr_misses"] == 4
    assert b.invalidate(buffers[0].data_ptr(), buffers[0].nbytes) == 1
    assert b.telemetry()["mr_entries"] == 1
    into(buffers[0])
    assert b.telemetry()["mr_misses"] == 5 and torch.equal(buffers[0], data)


def test_a_size_mismatch_is_an_error_not_an_overrun(fabric):
    for nbytes in (64, 100_000):                                       # eager and rendezvous
        f, (a, b) = fabric(eager_max=1024)
        data = torch.zeros(nbytes // 4)
        short = torch.zeros(nbytes // 8)
        r = b.recv(0, short.data_ptr(), short.nbytes, 3)
        a.send(1, data.data_ptr(), data.nbytes, 3)
        with pytest.raises(RuntimeError, match="met a receive of"):
            b.wait([r], soon())
        with pytest.raises(RuntimeError):
            b.recv(0, short.data_ptr(), short.nbytes, 4)               # broken stays broken


@pytest.mark.parametrize("fault,on,words", [("error", "send", "transport error"), ("corrupt", "send", "magic number"),
                                            ("error", "write", "transport error")])
def test_a_faulty_operation_breaks_the_endpoint_with_its_reason(fabric, fault, on, words):
    f, (a, b) = fabric(eager_max=1024)
    f.inject(fault, src=0, dst=1, on=on)
    data = torch.arange(50_000, dtype=torch.float32) if on == "write" else torch.arange(16, dtype=torch.float32)
    out = torch.zeros_like(data)
    r = b.recv(0, out.data_ptr(), out.nbytes, 1)
    s = a.send(1, data.data_ptr(), data.nbytes, 1)
    failures = []
    for endpoint, op in ((a, s), (b, r)):
        try:
            endpoint.wait([op], soon(1.0))
        except RuntimeError as exc:
            failures.append(str(exc))
    assert failures and any(words in text or "did not complete" in text for text in failures), failures
    broken = [e for e in (a, b) if e.telemetry()["broken"]]
    assert broken
    with pytest.raises(RuntimeError):
        broken[0].send(1 - broken[0].index, data.data_ptr(), 64, 2)


def test_a_lost_message_ends_in_the_deadline_not_a_hang(fabric):
    f, (a, b) = fabric()
    f.inject("drop", src=0, dst=1, on="send")
    out = torch.zeros(8)
    r = b.recv(0, out.data_ptr(), 32, 1)
    ones = torch.ones(8)
    a.send(1, ones.data_ptr(), 32, 1)
    began = time.monotonic()
    with pytest.raises(RuntimeError, match="did not complete within"):
        b.wait([r], soon(0.3))
    assert time.monotonic() - began < 2.0 and f.stats()["dropped"] == 1


def test_a_member_that_dies_fails_its_peers_operations(fabric):
    f, (a, b, c) = fabric(members=3)
    f.inject("kill", src=0, dst=1, on="send")                          # member 1 dies at the next send to it
    out = torch.zeros(8)
    waiting = a.recv(1, out.data_ptr(), 32, 5)
    ones = torch.ones(8)
    a.send(1, ones.data_ptr(), 32, 1)
    with pytest.raises(RuntimeError, match="flushed connection"):
        a.wait([waiting], soon(2.0))
    # members 0 and 2 were never wired to each other's failure: 2 still talks to nobody broken
    assert c.telemetry()["broken"] is False


def test_a_broken_receiver_revokes_its_registrations(fabric):
    f, (a, b) = fabric(eager_max=64, max_write=1000)
    data, out = torch.arange(10_000, dtype=torch.float32), torch.zeros(10_000)
    f.inject("delay", src=0, dst=1, on="write", nth=3, milliseconds=300)   # the sender stalls mid-message
    r = b.recv(0, out.data_ptr(), out.nbytes, 1)
    sender = threading.Thread(target=lambda: a.send(1, data.data_ptr(), data.nbytes, 1))
    sender.start()
    with pytest.raises(RuntimeError, match="did not complete within"):
        b.wait([r], soon(0.1))                                          # gives up while writes are still coming
    sender.join(5)
    time.sleep(0.5)
    assert a.telemetry()["broken"], "the late writes must have been refused"
    assert "refused remote access" in a.last_error()


def test_telemetry_counts_what_happened(fabric):
    f, (a, b) = fabric(eager_max=1024)
    exchange(a, b, torch.zeros(10))
    exchange(a, b, torch.zeros(10_000))
    t = a.telemetry()
    assert t["protocol"] == rdma.protocol_version() == 1 and t["member"] == 0 and t["members"] == 2
    assert (t["eager_sent"], t["rndv_sent"], t["bytes_sent"]) == (1, 1, 40 + 40_000)
    assert t["errors"] == 0 and t["pending_ops"] == 0 and not t["broken"]
    r = b.telemetry()
    assert (r["eager_recv"], r["rndv_recv"], r["bytes_recv"]) == (1, 1, 40 + 40_000)


def _expected(inputs, op):
    from gpubridge_b200.tagged import ring_order, segments
    fold = {"sum": torch.add, "max": torch.maximum}[op]
    members = len(inputs)
    if members == 2:
        return [fold(inputs[0], inputs[1]), fold(inputs[1], inputs[0])]
    out = torch.empty_like(inputs[0])
    for j, (start, length) in enumerate(segments(out.numel(), members)):
        order = ring_order(j, members)
        acc = inputs[order[0]][start:start + length].clone()
        for member in order[1:]:
            acc = fold(inputs[member][start:start + length], acc)
        out[start:start + length] = acc
    return [out] * members


@pytest.mark.parametrize("members", [2, 3, 4])
def test_collectives_ride_on_the_endpoint(fabric, members):
    from gpubridge_b200.tagged import DTYPE_CODES, OP_CODES
    f, endpoints = fabric(members=members, eager_max=2048, data_slots=4)
    cases = [(torch.float32, 10_000, "sum"), (torch.bfloat16, 1025, "sum"), (torch.int64, 3, "max"),
             (torch.float32, 70_000, "max")]
    inputs = {c: [(torch.randn(c[1], generator=torch.Generator().manual_seed(7 * r + c[1])) * 4).to(c[0])
                  for r in range(members)] for c in cases}
    got, errors = {}, []

    def member(rank):
        try:
            for seq, case in enumerate(cases, start=1):
                dtype, n, op = case
                t = inputs[case][rank].clone()
                endpoints[rank].all_reduce(t.data_ptr(), n, DTYPE_CODES[dtype], OP_CODES[op], 512, seq, soon(20))
                got[(rank, case)] = t
            t = torch.full((5000,), float(rank))
            endpoints[rank].broadcast(t.data_ptr(), t.nbytes, members - 1, 4096, 99, soon(20))
            got[(rank, "bcast")] = t
        except BaseException as exc:  # noqa: BLE001
            errors.append(exc)

    threads = [threading.Thread(target=member, args=(r,)) for r in range(members)]
    [t.start() for t in threads]
    [t.join(60) for t in threads]
    assert not errors, errors
    for case in cases:
        want = _expected(inputs[case], case[2])
        for rank in range(members):
            assert torch.equal(got[(rank, case)], want[rank]), (case, rank)
    assert all(float(got[(r, "bcast")][0]) == members - 1 for r in range(members))
    assert f.stats()["rnr"] == 0


def test_the_verbs_bridge_says_why_it_cannot_load():
    from gpubridge_b200.transport import resolve_transport
    with pytest.raises(ValueError, match="libibverbs"):
        resolve_transport("verbs")
    assert rdma.provider_available() is False


@pytest.mark.parametrize("mode", ["economy", "balanced", "latency"])
def test_progress_modes_deliver_the_same_messages(monkeypatch, mode):
    """How the progress thread waits (sleeping long, sleeping briefly, polling) is a setting of
    the process; every mode delivers, and the endpoint says which one it runs."""
    monkeypatch.setenv("GPUBRIDGE_VERBS_PROGRESS", mode)
    monkeypatch.setenv("GPUBRIDGE_VERBS_PROGRESS_CPU", "0")
    f = rdma.MockFabric(2)
    a, b = f.endpoint(0), f.endpoint(1)
    try:
        small, large = torch.arange(100, dtype=torch.float32), torch.arange(300_000, dtype=torch.float32)
        got_small, got_large = torch.zeros(100), torch.zeros(300_000)
        sends = [a.send(1, small.data_ptr(), small.nbytes, 1), a.send(1, large.data_ptr(), large.nbytes, 2)]
        recvs = [b.recv(0, got_small.data_ptr(), got_small.nbytes, 1), b.recv(0, got_large.data_ptr(), got_large.nbytes, 2)]
        b.wait(recvs, time.monotonic() + 10)
        a.wait(sends, time.monotonic() + 10)
        assert torch.equal(got_small, small) and torch.equal(got_large, large)
        told = a.telemetry()
        assert told["progress"] == mode and told["progress_cpu"] == 0
    finally:
        f.close()


def test_a_member_that_leaves_in_good_order_does_not_break_the_others():
    """Closing says goodbye first: the others stop reporting to the member that left, do not take
    the end of its link for a failure, and go on working among themselves; an operation that
    still expects something of it fails with the reason."""
    f = rdma.MockFabric(3)
    a, b, c = (f.endpoint(i, data_slots=4, ctrl_slots=3) for i in range(3))
    try:
        deadline = time.monotonic() + 10
        # enough traffic from a to b that b owes a credit reports
        payloads = [torch.full((64,), float(k)) for k in range(20)]
        outs = [torch.zeros(64) for _ in range(20)]
        recvs = [b.recv(0, o.data_ptr(), o.nbytes, 4) for o in outs]
        a.wait([a.send(1, p.data_ptr(), p.nbytes, 4) for p in payloads], deadline)
        b.wait(recvs, deadline)
        a.close()                                           # leaves while b and c go on
        f.endpoints.remove(a)
        time.sleep(0.2)
        big = torch.arange(200_000, dtype=torch.float32)
        got = torch.zeros(200_000)
        r = c.recv(1, got.data_ptr(), got.nbytes, 8)
        b.wait([b.send(2, big.data_ptr(), big.nbytes, 8)], deadline)
        c.wait([r], deadline)
        assert torch.equal(got, big)
        assert not b.telemetry()["broken"] and not c.telemetry()["broken"]
        # ... but nothing can be had from the member that left
        lost = torch.zeros(8)
        with pytest.raises(RuntimeError, match="left the bridge"):
            b.wait([b.recv(0, lost.data_ptr(), lost.nbytes, 9)], time.monotonic() + 5)
    finally:
        f.close()


def test_a_member_that_dies_without_a_word_still_breaks_its_peers():
    f = rdma.MockFabric(2)
    a, b = f.endpoint(0), f.endpoint(1)
    try:
        f.inject("kill", dst=1, nth=1)
        t, room = torch.ones(64), torch.zeros(64)
        # a small send is done for its caller once it is copied into a slot, so the wait also
        # covers a receive that only the dead member could have answered
        answer = a.recv(1, room.data_ptr(), room.nbytes, 2)
        with pytest.raises(RuntimeError):
            a.wait([a.send(1, t.data_ptr(), t.nbytes, 1), answer], time.monotonic() + 5)
        assert a.telemetry()["broken"]
    finally:
        f.close()


def test_close_waits_for_calls_that_are_inside_and_later_calls_are_refused(fabric):
    """Another thread is blocked in a wait when the endpoint is closed: the wait is ended with an
    error, the endpoint is freed only after that thread has left the library, and whatever is
    called afterwards raises instead of reaching freed memory."""
    f, (a, b) = fabric()
    room = torch.zeros(100)
    seen = {}

    def waits():
        try:
            a.wait([a.recv(1, room.data_ptr(), room.nbytes, 9)], soon(30))
            seen["wait"] = "returned"
        except RuntimeError as failure:
            seen["wait"] = str(failure)

    thread = threading.Thread(target=waits)
    thread.start()
    time.sleep(0.3)                                                 # it is inside the library now
    started = time.monotonic()
    a.close()
    thread.join(10)
    assert not thread.is_alive() and time.monotonic() - started < 8
    assert seen["wait"] != "returned" and "rdma endpoint" in seen["wait"]
    for call in (lambda: a.send(1, room.data_ptr(), 8, 1), lambda: a.recv(1, room.data_ptr(), 8, 1),
                 lambda: a.wait([1], soon(1)), a.telemetry, a.last_error):
        with pytest.raises(RuntimeError, match="closed"):
            call()
    a.abort()                                                       # harmless on a closed endpoint
    a.close()
    assert a.invalidate(room.data_ptr(), 8) == 0


@pytest.mark.parametrize("on", ["send", "write"])
def test_spurious_wake_ups_are_harmless(fabric, on):
    f, (a, b) = fabric(eager_max=1024, max_write=4096)
    for nth in (1, 2, 3, 5):
        f.inject("spurious", src=0, dst=1, on=on, nth=nth, milliseconds=7)          # seven empty wake-ups each
    small, large = torch.arange(100, dtype=torch.float32), torch.arange(50_000, dtype=torch.float32)
    for data in (small, large, small, large):
        out = torch.zeros_like(data)
        r = b.recv(0, out.data_ptr(), out.nbytes, 4)
        s = a.send(1, data.data_ptr(), data.nbytes, 4)
        a.wait([s], soon())
        b.wait([r], soon())
        assert torch.equal(out, data)
    assert not a.telemetry()["broken"] and not b.telemetry()["broken"]
    assert a.telemetry()["errors"] == 0 and b.telemetry()["pending_ops"] == 0


def test_a_completion_that_comes_after_the_peers_answer(fabric):
    """The send is delivered at once but the sender learns of it 300 ms later: by then the receiver
    has consumed the message and its credit (and, for a large message, its write grant) is back.
    Nothing may depend on the local completion coming first."""
    f, (a, b) = fabric(eager_max=1024, data_slots=2, max_write=4096)
    f.inject("late", src=0, dst=1, on="send", nth=1, milliseconds=300)
    data, out = torch.arange(200, dtype=torch.float32), torch.zeros(200)
    r = b.recv(0, out.data_ptr(), out.nbytes, 1)
    started = time.monotonic()
    s = a.send(1, data.data_ptr(), data.nbytes, 1)
    b.wait([r], soon())
    assert torch.equal(out, data) and time.monotonic() - started < 0.25              # the receiver did not wait for it
    a.wait([s], soon())                                # a small message is the endpoint's own copy: done for the caller
    before = a.telemetry()["completions"]
    time.sleep(0.45)
    assert a.telemetry()["completions"] == before + 1                                 # the held-back completion came in
    # and a large message whose request-to-send completes late still goes through, writes and all
    f.inject("late", src=0, dst=1, on="send", nth=1, milliseconds=200)
    f.inject("late", src=0, dst=1, on="write", nth=2, milliseconds=200)
    big, room = torch.arange(30_000, dtype=torch.float32), torch.zeros(30_000)
    r = b.recv(0, room.data_ptr(), room.nbytes, 2)
    s = a.send(1, big.data_ptr(), big.nbytes, 2)
    a.wait([s], soon())
    b.wait([r], soon())
    assert torch.equal(room, big)
    for _ in range(6):                                                                # credits are all back: a burst fits
        exchange(a, b, torch.ones(50))
    assert not a.telemetry()["broken"] and not b.telemetry()["broken"] and a.telemetry()["pending_ops"] == 0
