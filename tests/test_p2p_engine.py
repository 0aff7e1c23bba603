"""The point-to-point engine (gpubridge_b200/p2p.py) in one process: two or three engines
joined by an in-memory wire and an in-memory store, so every scenario runs in milliseconds and
failures can be injected exactly where wanted - a peer that never posts, a peer that dies with
a request on the wire, a descriptor that differs, a store that goes away.  The multi-process
tests (tests/test_p2p.py) cover the same engine over real Gloo."""
import threading
import time
from datetime import timedelta

import pytest
import torch

from gpubridge_b200 import p2p


class Store:
    """The part of a c10d store the engine uses, in memory and thread-safe."""

    def __init__(self):
        self.data, self.lock, self.broken = {}, threading.Lock(), False

    def _alive(self):
        if self.broken:
            raise RuntimeError("store connection lost")

    def set(self, key, value):
        self._alive()
        with self.lock:
            self.data[key] = value.encode() if isinstance(value, str) else value

    def get(self, key):
        self._alive()
        with self.lock:
            return self.data[key]

    def check(self, keys):
        self._alive()
        with self.lock:
            return all(k in self.data for k in keys)

    def delete_key(self, key):
        with self.lock:
            return self.data.pop(key, None) is not None

    def compare_set(self, key, expected, desired):
        self._alive()
        with self.lock:
            current = self.data.get(key)
            if current is None and expected == "":
                self.data[key] = desired.encode()
                return desired.encode()
            return current


class Request:
    def __init__(self):
        self.done, self.error = threading.Event(), None

    def wait(self, timeout=None):
        seconds = timeout.total_seconds() if isinstance(timeout, timedelta) else timeout
        if not self.done.wait(seconds):
            raise RuntimeError("wire request timed out")
        if self.error is not None:
            raise self.error
        return True

    def is_completed(self):
        return self.done.is_set()


class Wire:
    """Matches a send to the receive with the same (source, destination, tag), in posting order,
    and copies the bytes.  ``hold`` keeps matched pairs from completing until released;
    ``cut(rank)`` fails every request that involves that rank, now and later."""

    def __init__(self):
        self.lock = threading.Lock()
        self.waiting = {}                   # (src, dst, tag) -> [(sending, buffer, request)]
        self.dead, self.hold, self.held = set(), False, []
        self.log = []                        # (src, dst, tag, nbytes) of completed pairs, in order

    def link(self, rank):
        return _End(self, rank)

    def post(self, rank, buffer, peer, tag, sending):
        request = Request()
        key = (rank, peer, tag) if sending else (peer, rank, tag)
        with self.lock:
            if rank in self.dead or peer in self.dead:
                request.error = RuntimeError(f"connection to rank {peer} reset")
                request.done.set()
                return request
            queue = self.waiting.setdefault(key, [])
            if queue and queue[0][0] != sending:
                other_sending, other_buffer, other_request = queue.pop(0)
                src, dst = (buffer, other_buffer) if sending else (other_buffer, buffer)
                pair = (key, src, dst, request, other_request)
                if self.hold:
                    self.held.append(pair)
                else:
                    self._complete(pair)
            else:
                queue.append((sending, buffer, request))
        return request

    def _complete(self, pair):
        key, src, dst, a, b = pair
        if src.numel() != dst.numel():
            a.error = b.error = RuntimeError("wire: sizes differ (this would abort Gloo)")
        else:
            dst.copy_(src)
            self.log.append((*key, src.numel()))
        a.done.set()
        b.done.set()

    def release(self):
        with self.lock:
            self.hold = False
            for pair in self.held:
                self._complete(pair)
            self.held.clear()

    def cut(self, rank):
        with self.lock:
            self.dead.add(rank)
            for key, queue in self.waiting.items():
                if rank in key[:2]:
                    for _, _, request in queue:
                        request.error = RuntimeError(f"connection to rank {rank} reset")
                        request.done.set()
                    queue.clear()
            for pair in self.held:
                if rank in pair[0][:2]:
                    pair[3].error = pair[4].error = RuntimeError(f"connection to rank {rank} reset")
                    pair[3].done.set()
                    pair[4].done.set()
            self.held = [p for p in self.held if rank not in p[0][:2]]


class _End:
    def __init__(self, wire, rank):
        self.wire, self.rank, self.closed = wire, rank, False

    def post(self, buffer, peer, tag, sending):
        return self.wire.post(self.rank, buffer, peer, tag, sending)

    def close(self):
        self.closed = True


@pytest.fixture()
def pair():
    made = []

    def build(count=2, timeout=5.0, chunk_bytes=0, stores=None):
        wire = Wire()
        store = Store()
        engines = [p2p.Engine(wire.link(r), torch.device("cpu"), r, (stores or [store] * count)[r],
                              timedelta(seconds=timeout), chunk_bytes=chunk_bytes) for r in range(count)]
        made.extend(engines)
        return engines, wire, store

    yield build
    for engine in made:
        engine.close()


def test_a_message_arrives(pair):
    (a, b), wire, _ = pair()
    out = torch.zeros(100)
    recv = b.submit(out, 0, 3, False)
    send = a.submit(torch.arange(100.0), 1, 3, True)
    assert send.wait(5) and recv.wait(5)
    assert torch.equal(out, torch.arange(100.0))
    assert send.is_completed() and recv.exception() is None


@pytest.mark.parametrize("dtype", [torch.float32, torch.int64, torch.bfloat16, torch.uint8, torch.bool])
@pytest.mark.parametrize("n", [0, 1, 4099])
def test_any_dense_dtype_and_size_travels_as_bytes(pair, dtype, n):
    (a, b), _, _ = pair()
    data = (torch.arange(n) % 2).to(dtype) if dtype is torch.bool else (torch.arange(n) % 13).to(dtype)
    out = torch.zeros(n, dtype=dtype)
    works = [b.submit(out, 0, 0, False), a.submit(data, 1, 0, True)]
    [w.wait(5) for w in works]
    assert torch.equal(out, data)


def test_messages_of_one_lane_keep_their_order(pair):
    (a, b), wire, _ = pair()
    outs = [torch.zeros(8) for _ in range(20)]
    recvs = [b.submit(o, 0, 1, False) for o in outs]
    sends = [a.submit(torch.full((8,), float(i)), 1, 1, True) for i in range(20)]
    [w.wait(5) for w in sends + recvs]
    assert [float(o[0]) for o in outs] == [float(i) for i in range(20)]
    assert [entry[3] for entry in wire.log] == [32] * 20


def test_lanes_with_different_tags_do_not_wait_for_each_other(pair):
    (a, b), _, _ = pair()
    first, second = torch.zeros(4), torch.zeros(4)
    blocked = a.submit(torch.ones(4), 1, 101, True)            # its receive comes last
    quick = a.submit(torch.full((4,), 2.0), 1, 102, True)
    b.submit(second, 0, 102, False).wait(5)
    assert quick.wait(5) and not blocked.is_completed()
    b.submit(first, 0, 101, False).wait(5)
    assert blocked.wait(5) and float(first[0]) == 1.0 and float(second[0]) == 2.0


def test_send_and_receive_lanes_of_one_tag_are_separate(pair):
    (a, b), _, _ = pair()
    from_b, from_a = torch.zeros(4), torch.zeros(4)
    works = [a.submit(torch.full((4,), 5.0), 1, 7, True), a.submit(from_b, 1, 7, False),
             b.submit(torch.full((4,), 6.0), 0, 7, True), b.submit(from_a, 0, 7, False)]
    [w.wait(5) for w in works]
    assert float(from_b[0]) == 6.0 and float(from_a[0]) == 5.0


def test_three_ranks_route_by_peer(pair):
    (a, b, c), _, _ = pair(count=3)
    at_b, at_c = torch.zeros(3), torch.zeros(3)
    works = [a.submit(torch.full((3,), 1.0), 1, 0, True), a.submit(torch.full((3,), 2.0), 2, 0, True),
             b.submit(at_b, 0, 0, False), c.submit(at_c, 0, 0, False)]
    [w.wait(5) for w in works]
    assert float(at_b[0]) == 1.0 and float(at_c[0]) == 2.0


def test_chunked_transfer_sends_pieces_in_order_two_at_a_time(pair):
    (a, b), wire, _ = pair(chunk_bytes=64)
    data = torch.arange(100, dtype=torch.float32)              # 400 bytes: 6 pieces of 64, one of 16
    out = torch.zeros(100)
    wire.hold = True
    recv, send = b.submit(out, 0, 0, False), a.submit(data, 1, 0, True)
    time.sleep(0.2)
    assert len(wire.held) == 2, "at most two pieces of a transfer are on the wire"
    wire.release()
    recv.wait(5), send.wait(5)
    assert torch.equal(out, data)
    assert [entry[3] for entry in wire.log] == [64] * 6 + [16]


@pytest.mark.parametrize("theirs,what", [(torch.zeros(50), "size"), (torch.zeros(100, dtype=torch.int32), "dtype")])
def test_a_mismatch_raises_on_both_ends_and_nothing_is_posted(pair, theirs, what):
    (a, b), wire, _ = pair()
    send, recv = a.submit(torch.zeros(100), 1, 5, True), b.submit(theirs, 0, 5, False)
    for work in (send, recv):
        with pytest.raises(RuntimeError, match="mismatch"):
            work.wait(5)
    assert not wire.log and not wire.waiting.get((0, 1, 5))


def test_chunk_setting_is_part_of_the_agreement():
    wire, store = Wire(), Store()
    a = p2p.Engine(wire.link(0), torch.device("cpu"), 0, store, timedelta(seconds=5), chunk_bytes=64)
    b = p2p.Engine(wire.link(1), torch.device("cpu"), 1, store, timedelta(seconds=5), chunk_bytes=0)
    try:
        send, recv = a.submit(torch.zeros(100), 1, 0, True), b.submit(torch.zeros(100), 0, 0, False)
        with pytest.raises(RuntimeError, match="mismatch"):
            send.wait(5)
        with pytest.raises(RuntimeError, match="mismatch"):
            recv.wait(5)
    finally:
        a.close(), b.close()


def test_a_peer_that_never_posts_runs_into_the_deadline(pair):
    (a, b), _, _ = pair(timeout=0.4)
    began = time.monotonic()
    work = a.submit(torch.zeros(10), 1, 9, True)
    with pytest.raises(RuntimeError, match="timed out"):
        work.wait(5)
    assert 0.3 < time.monotonic() - began < 2.0


def test_the_deadline_counts_time_spent_queued(pair):
    (a, b), _, _ = pair(timeout=0.5)
    head = a.submit(torch.zeros(10), 1, 2, True)                 # never matched: blocks its lane
    behind = a.submit(torch.zeros(10), 1, 2, True)               # never even starts
    began = time.monotonic()
    with pytest.raises(RuntimeError, match="timed out"):
        behind.wait(5)
    assert time.monotonic() - began < 2.0
    with pytest.raises(RuntimeError):
        head.wait(5)


def test_one_failure_fails_every_pending_handle_here_and_there(pair):
    (a, b), _, store = pair(timeout=0.4)
    other_lane = b.submit(torch.zeros(4), 0, 77, False)          # pending on the healthy side
    doomed = a.submit(torch.zeros(4), 1, 1, True)                # times out on rank 0
    with pytest.raises(RuntimeError, match="timed out"):
        doomed.wait(5)
    assert store.check(["failure"]) and b"rank 0" in store.get("failure")
    with pytest.raises(RuntimeError, match="rank 0"):            # rank 1 learns of it from the store
        other_lane.wait(5)
    for engine in (a, b):
        with pytest.raises(RuntimeError):
            engine.submit(torch.zeros(4), 1 - engine.rank, 0, True)


def test_only_the_first_failure_is_published(pair):
    (a, b), _, store = pair(timeout=0.3)
    first = a.submit(torch.zeros(4), 1, 1, True)
    with pytest.raises(RuntimeError):
        first.wait(5)
    record = store.get("failure")
    with pytest.raises(RuntimeError):
        b.submit(torch.zeros(4), 0, 2, True).wait(5)
    assert store.get("failure") == record


def test_a_peer_that_dies_mid_transfer_fails_the_survivor(pair):
    (a, b), wire, _ = pair(chunk_bytes=64)
    wire.hold = True
    send, recv = a.submit(torch.zeros(1000), 1, 0, True), b.submit(torch.zeros(1000), 0, 0, False)
    time.sleep(0.2)
    assert wire.held
    wire.cut(1)                                                   # rank 1 goes away
    with pytest.raises(RuntimeError, match="reset"):
        send.wait(5)
    with pytest.raises(RuntimeError):
        a.submit(torch.zeros(4), 1, 3, True)


def test_losing_the_store_fails_pending_work(pair):
    stores = [Store(), Store()]
    (a, b), _, _ = pair(stores=stores, timeout=5)
    pending = a.submit(torch.zeros(4), 1, 0, True)
    time.sleep(0.1)
    stores[0].broken = True
    with pytest.raises(RuntimeError, match="store"):
        pending.wait(5)


def test_close_fails_what_is_pending_and_returns_quickly(pair):
    (a, b), _, _ = pair(timeout=30)
    pending = [a.submit(torch.zeros(4), 1, t, True) for t in range(5)]
    began = time.monotonic()
    a.close()
    assert time.monotonic() - began < 1.0
    for work in pending:
        with pytest.raises(RuntimeError, match="destroyed"):
            work.wait(1)
    with pytest.raises(RuntimeError, match="destroyed"):
        a.submit(torch.zeros(4), 1, 0, True)
    a.close()                                                      # twice is fine
    assert a.link.closed


def test_a_future_callback_may_wait_on_another_handle(pair):
    (a, b), _, _ = pair()
    first_out, second_out, seen = torch.zeros(4), torch.zeros(4), []
    first = b.submit(first_out, 0, 1, False)
    second = b.submit(second_out, 0, 2, False)

    def after_first(future):
        second.wait(5)                                             # would deadlock on the engine's own loop
        seen.append((float(future.value()[0][0]), float(second_out[0])))

    first.get_future().then(after_first)
    a.submit(torch.full((4,), 1.0), 1, 1, True)
    a.submit(torch.full((4,), 2.0), 1, 2, True)
    deadline = time.monotonic() + 5
    while not seen and time.monotonic() < deadline:
        time.sleep(0.01)
    assert seen == [(1.0, 2.0)]


def test_futures_carry_the_tensor_or_the_error(pair):
    (a, b), _, _ = pair(timeout=0.3)
    out = torch.zeros(4)
    recv = b.submit(out, 0, 0, False)
    a.submit(torch.ones(4), 1, 0, True).wait(5)
    recv.wait(5)
    recv.get_future().wait()
    assert recv.get_future().value()[0] is out
    late = a.submit(torch.zeros(4), 1, 9, True)
    with pytest.raises(RuntimeError):
        late.wait(5)
    with pytest.raises(Exception):
        late.get_future().wait()


def test_many_lanes_at_once(pair):
    (a, b), _, _ = pair()
    outs = {tag: torch.zeros(16) for tag in range(40)}
    works = [b.submit(outs[tag], 0, tag, False) for tag in range(40)]
    works += [a.submit(torch.full((16,), float(tag)), 1, tag, True) for tag in reversed(range(40))]
    [w.wait(5) for w in works]
    assert all(float(outs[tag][0]) == float(tag) for tag in range(40))
    assert not a._lanes and not b._lanes, "finished lanes are forgotten"


def test_submissions_from_several_threads(pair):
    (a, b), _, _ = pair()
    outs = [[torch.zeros(4) for _ in range(10)] for _ in range(4)]
    errors = []

    def sender(tag):
        try:
            [a.submit(torch.full((4,), float(i)), 1, tag, True).wait(5) for i in range(10)]
        except BaseException as exc:  # noqa: BLE001
            errors.append(exc)

    def receiver(tag):
        try:
            [b.submit(outs[tag][i], 0, tag, False).wait(5) for i in range(10)]
        except BaseException as exc:  # noqa: BLE001
            errors.append(exc)

    threads = [threading.Thread(target=f, args=(t,)) for t in range(4) for f in (sender, receiver)]
    [t.start() for t in threads]
    [t.join(10) for t in threads]
    assert not errors
    assert all([float(o[0]) for o in outs[t]] == [float(i) for i in range(10)] for t in range(4))


def test_handshake_keys_do_not_pile_up_in_the_store(pair):
    (a, b), _, store = pair()
    for i in range(10):
        out = torch.zeros(4)
        works = [b.submit(out, 0, 0, False), a.submit(torch.ones(4), 1, 0, True)]
        [w.wait(5) for w in works]
    assert not [k for k in store.data if k != "failure"], store.data.keys()


def test_chunk_bytes_setting(monkeypatch):
    monkeypatch.delenv(p2p.CHUNK_BYTES_ENV, raising=False)
    assert p2p.chunk_bytes_setting() == 0
    monkeypatch.setenv(p2p.CHUNK_BYTES_ENV, "64K")
    assert p2p.chunk_bytes_setting() == 65536
    for bad in ("12", "0", "-8"):
        monkeypatch.setenv(p2p.CHUNK_BYTES_ENV, bad)
        with pytest.raises(ValueError):
            p2p.chunk_bytes_setting()


def test_torch_work_adapter(pair):
    (a, b), _, _ = pair()
    out = torch.zeros(4)
    inner = b.submit(out, 0, 0, False)
    work = p2p.TorchWork(inner, 0)
    assert not work.is_completed() and not work.is_success()
    a.submit(torch.ones(4), 1, 0, True).wait(5)
    assert work.wait(timedelta(seconds=5)) and work.is_completed() and work.is_success()
    assert work.exception() is None and work._source_rank() == 0
    work.synchronize()
    assert work.get_future() is inner.get_future()
