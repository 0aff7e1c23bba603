"""Point-to-point between islands through host memory: one event loop, a small wire pool.

On a B200 box every send / recv is an NCCL p2p call (:mod:`gpubridge_b200.torch_backend`); this
module is the other route - CPU simulation, and ranks on different machines - where the bytes
travel over the job's Gloo communicator.  What a user of the reference's engine relies on
(src/gpubridge/p2p.py, docs/TORCH_BACKEND.md "Point-to-point") holds here too, by a different
construction:

==============================  ===============================================================
guarantee                        how it is kept here
==============================  ===============================================================
messages of one (peer, tag,      every such *lane* is a FIFO of :class:`Transfer` state
direction) never overtake        machines; only the head of a lane is ever advanced
lanes do not block each other    one loop thread polls the heads of all lanes round-robin and
                                 nothing in a step blocks: stores are probed, CUDA events
                                 queried, and a posted Gloo request - which only completes
                                 inside its own ``wait`` - is waited for by a pool of daemon
                                 threads that grows with the requests in flight
a size / dtype mismatch raises   before any payload is posted the two ends swap a descriptor
instead of aborting in Gloo      through the store and compare it
an operation's deadline covers   the deadline is fixed at ``submit`` and checked on every step
its time in the queue            of the machine, queued or not
one failure fails everything,    the first error is written once to the store's ``failure``
on both ends                     key (``compare_set``); the loop probes that key every 50 ms
                                 while work is pending and fails all local handles
futures resolve off the engine   a second thread runs ``set_result`` / callbacks, so a callback
                                 may itself wait on a handle
teardown never waits for a peer  ``close`` fails what is pending, stops the loop and joins it
                                 for at most 200 ms
==============================  ===============================================================

CPU tensors are sent from and received into their own memory (chunks are views).  CUDA
tensors go through pinned slots, two per transfer, with copies on the engine's own streams
ordered by events, so a copy overlaps the wire time of the other slot.
"""
from __future__ import annotations

import collections
import contextlib
import json
import os
import queue
import threading
import time
from datetime import timedelta

import torch
import torch.distributed as dist

from gpubridge_b200.config import parse_size
from gpubridge_b200.groups import Comm
from gpubridge_b200.work import Work

CHUNK_BYTES_ENV = "GPUBRIDGE_P2P_CHUNK_BYTES"
HEALTH_PERIOD = 0.05                 # seconds between probes of the shared failure key
IDLE_NAP = (50e-6, 2e-3)             # the loop's back-off when no head made progress
TEARDOWN_LIMIT = 0.2


def chunk_bytes_setting() -> int:
    """``GPUBRIDGE_P2P_CHUNK_BYTES``: 0 (unset) sends a tensor as one message; otherwise the
    size of a piece, a positive multiple of 8 bytes."""
    text = os.environ.get(CHUNK_BYTES_ENV, "").strip()
    if not text:
        return 0
    size = parse_size(text)
    if size <= 0 or size % 8:
        raise ValueError(f"{CHUNK_BYTES_ENV} must be a positive multiple of 8 bytes")
    return size


class TorchWork(dist.Work):
    """Adapter: what ``torch.distributed`` hands its callers, backed by a library handle (so
    ``wait`` raises the Python exception and honours a host timeout)."""

    def __init__(self, inner: Work, source_rank: int) -> None:
        super().__init__()
        self._inner, self._source = inner, source_rank

    def wait(self, timeout=None) -> bool:
        return self._inner.wait(timeout)

    def synchronize(self) -> None:
        self._inner.wait()

    def is_completed(self) -> bool:
        return self._inner.is_completed()

    def is_success(self) -> bool:
        return self._inner.is_completed() and self._inner.exception() is None

    def exception(self):
        return self._inner.exception()

    def get_future(self):
        return self._inner.get_future()

    def _source_rank(self) -> int:
        return self._source


class GlooLink:
    """Byte messages over a Gloo communicator that spans every rank of the job."""

    def __init__(self, group: Comm) -> None:
        self.group = group

    def post(self, buffer: torch.Tensor, peer: int, tag: int, sending: bool):
        return self.group.send(buffer, peer, tag) if sending else self.group.recv(buffer, peer, tag)

    def close(self) -> None:
        pass


class _Ticket(Work):
    """A handle whose completion and whose future are settled by different threads."""

    def _finish(self, error):
        self._error = error
        self._done.set()


class _Piece:
    """One chunk of a transfer in flight: its wire request and, for CUDA, its slot and copy."""
    __slots__ = ("view", "host", "request", "copied", "arrived", "error")

    def __init__(self, view, host):
        self.view, self.host, self.request, self.copied = view, host, None, None
        self.arrived, self.error = False, None

    def wire_done(self) -> bool:
        if self.error is not None:
            raise self.error
        return self.arrived


class _WirePool:
    """Daemon threads that sit in ``request.wait()`` so the loop never has to.  A Gloo send or
    receive completes once the peer has posted the other half, which the peer does from its
    own loop, never from its pool - so a full pool delays, but cannot deadlock."""

    def __init__(self, most: int = 16) -> None:
        self.most, self.idle, self.threads = most, 0, 0
        self.jobs: queue.SimpleQueue = queue.SimpleQueue()
        self.lock = threading.Lock()

    def watch(self, piece: _Piece, deadline: float) -> None:
        with self.lock:
            if self.idle == 0 and self.threads < self.most:
                self.threads += 1
                threading.Thread(target=self._serve, name="gpubridge-p2p-wire", daemon=True).start()
        self.jobs.put((piece, deadline))

    def _serve(self) -> None:
        while True:
            with self.lock:
                self.idle += 1
            job = self.jobs.get()
            with self.lock:
                self.idle -= 1
            if job is None:
                return
            piece, deadline = job
            try:
                piece.request.wait(timedelta(seconds=max(0.001, deadline - time.monotonic())))
                piece.arrived = True
            except BaseException as failure:  # noqa: BLE001 - handed to the loop
                piece.error = failure

    def stop(self) -> None:
        with self.lock:
            count = self.threads
        for _ in range(count):
            self.jobs.put(None)


class Transfer:
    """A send or a receive as a state machine: ``queued`` (waiting for the producer's CUDA
    event) -> ``offered`` (descriptor published, waiting for the peer's) -> ``moving`` (pieces
    on the wire, at most two) -> finished.  :meth:`step` never blocks and returns True when it
    changed something."""

    def __init__(self, engine: "Engine", ticket: _Ticket, tensor: torch.Tensor, peer: int, tag: int,
                 sending: bool, number: int, deadline: float, ready) -> None:
        self.engine, self.ticket, self.tensor = engine, ticket, tensor
        self.peer, self.tag, self.sending, self.number = peer, tag, sending, number
        self.deadline, self.ready = deadline, ready
        self.state = "queued"
        self.bytes = tensor.reshape(-1).view(torch.uint8)
        size = engine.chunk_bytes or max(1, self.bytes.numel())
        self.views = list(self.bytes.split(size)) if self.bytes.numel() else [self.bytes]
        self.next_piece = 0
        self.flying: collections.deque[_Piece] = collections.deque()
        self.slots: list[torch.Tensor] = []
        self.last_copy = None
        where = (engine.rank, peer) if sending else (peer, engine.rank)
        self.key = f"{where[0]}/{where[1]}/{tag}/{number}"
        self.what = f"point-to-point {'send' if sending else 'recv'} with rank {peer}, tag {tag}"

    # -- the machine ---------------------------------------------------------------------------------
    def step(self) -> bool:
        if time.monotonic() >= self.deadline:
            waited = "in queue" if self.state == "queued" else "waiting for its peer"
            raise TimeoutError(f"{self.what} timed out {waited}")
        return getattr(self, "_" + self.state)()

    def _queued(self) -> bool:
        if self.ready is not None and not self.ready.query():
            return False
        mine = "send" if self.sending else "recv"
        self.engine.store.set(f"{self.key}/{mine}", self._descriptor())
        self.state = "offered"
        return True

    def _descriptor(self) -> str:
        return json.dumps([self.bytes.numel(), str(self.tensor.dtype), self.engine.chunk_bytes])

    def _offered(self) -> bool:
        theirs = f"{self.key}/{'recv' if self.sending else 'send'}"
        store = self.engine.store
        if not store.check([theirs]):
            return False
        other = store.get(theirs).decode()
        store.delete_key(theirs)
        if other != self._descriptor():
            raise ValueError(f"point-to-point payload mismatch with rank {self.peer}, tag {self.tag}: "
                             f"local {self._descriptor()}, peer {other}")
        if self.tensor.device.type == "cuda":
            size = max(v.numel() for v in self.views)
            self.slots = [torch.empty(max(1, size), dtype=torch.uint8, pin_memory=True)
                          for _ in range(min(2, len(self.views)))]
            self.tensor.record_stream(self.engine.copy_stream(self.tensor.device))
        self.state = "moving"
        return True

    def _moving(self) -> bool:
        moved = False
        on_gpu = bool(self.slots)
        # retire the oldest piece (pieces of one transfer complete in order on one Gloo tag)
        while self.flying:
            piece = self.flying[0]
            if self.sending:
                if piece.request is None:                       # still being copied to its slot
                    if not piece.copied.query():
                        break
                    self._post(piece)
                    moved = True
                if not piece.wire_done():                       # raises what the wire raised
                    break
            else:
                if piece.copied is None:
                    if not piece.wire_done():
                        break
                    if on_gpu:
                        piece.copied = self._copy(piece.view, piece.host)
                        self.last_copy = piece.copied
                        moved = True
                if on_gpu and not piece.copied.query():
                    break
            self.flying.popleft()
            moved = True
        # launch pieces while a slot (GPU) or the two-in-flight budget (CPU) allows
        while self.next_piece < len(self.views) and len(self.flying) < 2:
            view = self.views[self.next_piece]
            host = self.slots[self.next_piece % 2][:view.numel()] if on_gpu else view
            piece = _Piece(view, host)
            if self.sending:
                if on_gpu:
                    piece.copied = self._copy(host, view)
                else:
                    self._post(piece)
            else:
                self._post(piece)
            self.flying.append(piece)
            self.next_piece += 1
            moved = True
        if self.next_piece == len(self.views) and not self.flying:
            self.state = "finished"
        return moved

    def _post(self, piece: _Piece) -> None:
        piece.request = self.engine.link.post(piece.host, self.peer, self.tag, self.sending)
        self.engine.wire.watch(piece, self.deadline)

    def _copy(self, dst: torch.Tensor, src: torch.Tensor):
        stream = self.engine.copy_stream(self.tensor.device)
        with torch.cuda.stream(stream):
            dst.copy_(src, non_blocking=True)
            done = torch.cuda.Event()
            done.record(stream)
        return done

    def _finished(self) -> bool:
        return False


class Engine:
    """All cross-island point-to-point traffic of one process group."""

    def __init__(self, link, device: torch.device, rank: int, store, timeout: timedelta | None, *,
                 pinned: bool = False, chunk_bytes: int = 0) -> None:
        self.link, self.device, self.rank, self.store = link, device, rank, store
        self.limit = (timeout or timedelta(minutes=30)).total_seconds()
        self.chunk_bytes = chunk_bytes
        self.pinned = pinned                       # CUDA tensors always use pinned slots here
        self._guard = threading.Lock()
        self._lanes: dict[tuple[int, int, bool], collections.deque[Transfer]] = {}
        self._numbers: collections.Counter = collections.Counter()
        self._broken: BaseException | None = None
        self._closing = False
        self._work_arrived = threading.Event()
        self._settled: queue.SimpleQueue = queue.SimpleQueue()
        self.wire = _WirePool()
        self._streams: dict[torch.device, torch.cuda.Stream] = {}
        self._callback_streams: dict[torch.device, torch.cuda.Stream] = {}
        self._loop_thread = threading.Thread(target=self._loop, name="gpubridge-p2p-loop", daemon=True)
        self._callback_thread = threading.Thread(target=self._callbacks, name="gpubridge-p2p-futures",
                                                 daemon=True)
        self._loop_thread.start()
        self._callback_thread.start()

    def copy_stream(self, device: torch.device) -> torch.cuda.Stream:
        stream = self._streams.get(device)
        if stream is None:
            stream = self._streams[device] = torch.cuda.Stream(device)
        return stream

    # -- public ----------------------------------------------------------------------------------------
    def check(self) -> None:
        """Raise if the group was destroyed, failed here, or failed on the other end."""
        with self._guard:
            if self._closing:
                raise RuntimeError("gpubridge point-to-point group was destroyed")
            if self._broken is not None:
                raise RuntimeError(f"gpubridge point-to-point group failed: {self._broken}")
        if self.store.check(["failure"]):
            remote = RuntimeError(self.store.get("failure").decode())
            self._break(remote, announce=False)
            raise remote

    def submit(self, tensor: torch.Tensor, peer: int, tag: int, sending: bool) -> Work:
        self.check()
        ready = None
        if tensor.device.type == "cuda":
            ready = torch.cuda.Event()
            ready.record(torch.cuda.current_stream(tensor.device))
        ticket = _Ticket("send" if sending else "recv", tensor.device, [tensor])
        lane_key = (peer, tag, sending)
        with self._guard:
            if self._closing or self._broken is not None:
                raise RuntimeError("gpubridge point-to-point group is not usable any more")
            number = self._numbers[lane_key]
            self._numbers[lane_key] += 1
            transfer = Transfer(self, ticket, tensor, peer, tag, sending, number,
                                time.monotonic() + self.limit, ready)
            self._lanes.setdefault(lane_key, collections.deque()).append(transfer)
        self._work_arrived.set()
        return ticket

    def close(self, timeout: float = TEARDOWN_LIMIT) -> None:
        with self._guard:
            if self._closing:
                return
            self._closing = True
            orphans = [t for lane in self._lanes.values() for t in lane]
            self._lanes.clear()
        self._settle(orphans, RuntimeError("point-to-point group was destroyed"))
        self._work_arrived.set()
        self._settled.put(None)
        self.wire.stop()
        self._loop_thread.join(timeout)
        self.link.close()

    # -- the loop --------------------------------------------------------------------------------------
    def _heads(self) -> list[Transfer]:
        with self._guard:
            return [lane[0] for lane in self._lanes.values() if lane]

    def _retire(self, transfer: Transfer) -> None:
        key = (transfer.peer, transfer.tag, transfer.sending)
        with self._guard:
            lane = self._lanes.get(key)
            if not lane or lane[0] is not transfer:
                return                                          # already failed or closed
            lane.popleft()
            if not lane:
                del self._lanes[key]
        if transfer.last_copy is not None:
            transfer.ticket._event = transfer.last_copy          # wait() orders the caller's stream
        self._settle([transfer], None)

    def _loop(self) -> None:
        nap, next_probe = IDLE_NAP[0], 0.0
        while True:
            heads = self._heads()
            if self._closing:
                return
            if not heads:
                self._work_arrived.clear()
                if not self._heads() and not self._closing:
                    self._work_arrived.wait()
                nap = IDLE_NAP[0]
                continue
            progressed = False
            try:
                now = time.monotonic()
                if now >= next_probe:
                    next_probe = now + HEALTH_PERIOD
                    if self.store.check(["failure"]):
                        raise _Remote(self.store.get("failure").decode())
                for transfer in heads:
                    if transfer.step():
                        progressed = True
                    if transfer.state == "finished":
                        self._retire(transfer)
            except _Remote as told:
                self._break(RuntimeError(str(told)), announce=False)
                return
            except BaseException as failure:  # noqa: BLE001 - every pending handle hears of it
                self._break(failure, announce=True)
                return
            if progressed:
                nap = IDLE_NAP[0]
            else:
                time.sleep(nap)
                nap = min(2 * nap, IDLE_NAP[1])

    def _break(self, error: BaseException, *, announce: bool) -> None:
        with self._guard:
            if self._broken is not None or self._closing:
                return
            self._broken = error
            victims = [t for lane in self._lanes.values() for t in lane]
            self._lanes.clear()
        if announce:
            with contextlib.suppress(Exception):
                self.store.compare_set("failure", "", f"rank {self.rank}: {error}")
        self._settle(victims, error)

    def _settle(self, transfers, error) -> None:
        for transfer in transfers:
            transfer.ticket._finish(error)
            self._settled.put(transfer.ticket)

    # -- futures ---------------------------------------------------------------------------------------
    def _callbacks(self) -> None:
        while True:
            ticket = self._settled.get()
            if ticket is None:
                return
            scope = contextlib.nullcontext()
            if ticket._event is not None:
                stream = self._callback_streams.get(ticket._device)
                if stream is None:
                    stream = self._callback_streams[ticket._device] = torch.cuda.Stream(ticket._device)
                stream.wait_event(ticket._event)
                scope = torch.cuda.stream(stream)
            with scope:
                if ticket._error is None:
                    ticket._future.set_result(ticket._result)
                else:
                    ticket._future.set_exception(ticket._error)


class _Remote(Exception):
    """The other end published a failure."""
