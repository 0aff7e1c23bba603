"""Cross-island point-to-point for the torch backend (host-staged route).

On a GPU box every send/recv, same island or not, is an NCCL p2p call overlapped with
compute (:mod:`gpubridge_b200.torch_backend`).  This engine is the other route - CPU
simulation and the cross-node fallback - with the reference's guarantees
(src/gpubridge/p2p.py:57-439, docs/TORCH_BACKEND.md:401-445):

* one lane (thread, stream, FIFO) per ``(peer, tag, direction)``, a sequence number per
  lane, so messages of one lane never overtake each other and lanes never block each other;
* a handshake on the store (``[nbytes, dtype, chunk]`` as JSON) *before* the payload is
  posted, because Gloo aborts the process on a size mismatch; a mismatch raises instead;
* every operation has a deadline that includes its time in the queue;
* a failure is published once with ``compare_set("failure", ...)``; a watcher polls it
  every 50 ms, only while operations are pending, and fails every pending handle;
* completion is published by the lane itself, futures are resolved by one completion
  thread, so a callback may wait on any handle;
* teardown is bounded (200 ms) and never waits for a missing peer.
"""
from __future__ import annotations

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
from gpubridge_b200.staging import make_staging
from gpubridge_b200.work import Work

CHUNK_BYTES_ENV = "GPUBRIDGE_P2P_CHUNK_BYTES"
MATCH_POLL_FIRST = 50e-6
MATCH_POLL_MAX = 0.002
WATCH_INTERVAL = 0.05


def chunk_bytes_setting() -> int:
    """0: one message per tensor; >0: two staging slots of that size."""
    raw = os.environ.get(CHUNK_BYTES_ENV, "").strip()
    if not raw:
        return 0
    size = parse_size(raw)
    if size < 8 or size % 8:
        raise ValueError(f"{CHUNK_BYTES_ENV} must be a positive multiple of 8 bytes")
    return size


class TorchWork(dist.Work):
    """A ``torch.distributed.Work`` that delegates to a library :class:`Work`, keeping the
    Python exception and the optional host timeout of ``wait``."""

    def __init__(self, work: Work, source: int) -> None:
        super().__init__()
        self.work, self.source = work, source

    def wait(self, timeout=None) -> bool:
        return self.work.wait(timeout)

    def is_completed(self) -> bool:
        return self.work.is_completed()

    def is_success(self) -> bool:
        return self.is_completed() and self.work.exception() is None

    def get_future(self):
        return self.work.get_future()

    def exception(self):
        return self.work.exception()

    def synchronize(self) -> None:
        self.wait()

    def _source_rank(self) -> int:
        return self.source


class _Handle(Work):
    """Completion is published by the lane; the future is resolved by the completer."""

    def _finish(self, error):
        self._error = error
        self._done.set()


class GlooLink:
    """Raw bytes over an existing Gloo communicator of every member."""

    def __init__(self, group: Comm) -> None:
        self.group = group

    def post(self, tensor: torch.Tensor, peer: int, tag: int, sending: bool):
        return (self.group.send if sending else self.group.recv)(tensor, peer, tag)

    def close(self) -> None:
        pass


class Engine:
    def __init__(self, link, device: torch.device, rank: int, store,
                 timeout: timedelta | None, *, pinned: bool = False, chunk_bytes: int = 0):
        self.link, self.device, self.rank, self.store = link, device, rank, store
        self.timeout = (timeout or timedelta(minutes=30)).total_seconds()
        self.pinned, self.chunk_bytes = pinned, chunk_bytes
        self._lock = threading.RLock()
        self._lanes: dict[tuple[int, int, bool], _Lane] = {}
        self._next: dict[tuple[int, int, bool], int] = {}
        self._pending: dict[_Handle, None] = {}
        self._closed = False
        self._failed: BaseException | None = None
        self._resolve_queue: queue.SimpleQueue = queue.SimpleQueue()
        self._streams: dict[torch.device, torch.cuda.Stream] = {}
        self._stop, self._wake = threading.Event(), threading.Event()
        for target, name in ((self._resolver, "gpubridge-p2p-completion"),
                             (self._watch, "gpubridge-p2p-health")):
            threading.Thread(target=target, name=name, daemon=True).start()

    # -- background threads --------------------------------------------------------------------
    def _resolver(self) -> None:
        while True:
            handle = self._resolve_queue.get()
            if handle is None:
                return
            scope = contextlib.nullcontext()
            if handle._event is not None:
                stream = self._streams.setdefault(handle._device,
                                                  torch.cuda.Stream(handle._device))
                stream.wait_event(handle._event)
                scope = torch.cuda.stream(stream)
            with scope:
                if handle._error is None:
                    handle._future.set_result(handle._result)
                else:
                    handle._future.set_exception(handle._error)
            del handle

    def _watch(self) -> None:
        while not self._stop.is_set():
            with self._lock:
                if self._closed:
                    return
                idle = not self._pending
                if idle:
                    self._wake.clear()
            if idle:
                self._wake.wait()
                continue
            if self._stop.wait(WATCH_INTERVAL - time.monotonic() % WATCH_INTERVAL):
                return
            try:
                self.check()
            except BaseException as exc:  # noqa: BLE001 - store loss fails pending handles too
                self._fail(exc, publish=False)
                return

    # -- state -----------------------------------------------------------------------------------
    def check(self) -> None:
        with self._lock:
            if self._closed:
                raise RuntimeError("gpubridge point-to-point group was destroyed")
            if self._failed is not None:
                raise RuntimeError(f"gpubridge point-to-point group failed: {self._failed}")
        if self.store.check(["failure"]):
            error = RuntimeError(self.store.get("failure").decode())
            self._fail(error, publish=False)
            raise error

    def _settle(self, handles, error) -> None:
        for handle in handles:
            handle._finish(error)
            self._resolve_queue.put(handle)

    def _done(self, handle, error=None) -> None:
        with self._lock:
            if handle not in self._pending:
                return
            del self._pending[handle]
        self._settle([handle], error)

    def _fail(self, error: BaseException, *, publish: bool = True) -> None:
        with self._lock:
            if self._failed is not None or self._closed:
                return
            self._failed = error
            if publish:
                with contextlib.suppress(Exception):
                    self.store.compare_set("failure", "", f"rank {self.rank}: {error}")
            pending = list(self._pending)
            self._pending.clear()
        self._settle(pending, error)

    # -- API -------------------------------------------------------------------------------------
    def submit(self, tensor: torch.Tensor, peer: int, tag: int, sending: bool) -> Work:
        self.check()
        ready = None
        if tensor.device.type == "cuda":
            ready = torch.cuda.Event()
            ready.record(torch.cuda.current_stream(tensor.device))
        handle = _Handle("send" if sending else "recv", tensor.device, [tensor])
        with self._lock:
            self.check()
            key = (peer, tag, sending)
            seq = self._next.get(key, 0)
            self._next[key] = seq + 1
            lane = self._lanes.get(key)
            if lane is None:
                lane = self._lanes[key] = _Lane(self, peer, tag, sending)
            self._pending[handle] = None
            lane.queue.put((handle, tensor, ready, time.monotonic() + self.timeout, seq))
        self._wake.set()
        return handle

    def match(self, tensor, peer, tag, seq, sending, deadline) -> None:
        """Agree with the peer on size, dtype and chunking before any payload moves."""
        self.check()
        if time.monotonic() >= deadline:
            raise TimeoutError(f"point-to-point operation with rank {peer} timed out in queue")
        src, dst = (self.rank, peer) if sending else (peer, self.rank)
        mine, theirs = ("send", "recv") if sending else ("recv", "send")
        base = f"{src}/{dst}/{tag}/{seq}"
        descriptor = json.dumps([tensor.numel() * tensor.element_size(), str(tensor.dtype),
                                 self.chunk_bytes])
        self.store.set(f"{base}/{mine}", descriptor)
        key = f"{base}/{theirs}"
        late = f"point-to-point {mine} with rank {peer}, tag {tag} timed out"
        pause = MATCH_POLL_FIRST
        while not self.store.check([key]):
            self.check()
            left = deadline - time.monotonic()
            if left <= 0:
                raise TimeoutError(late)
            time.sleep(min(pause, left))
            pause = min(2 * pause, MATCH_POLL_MAX)
        other = self.store.get(key).decode()
        self.store.delete_key(key)
        if time.monotonic() >= deadline:
            raise TimeoutError(late)
        if other != descriptor:
            raise ValueError(f"point-to-point payload mismatch with rank {peer}, tag {tag}: "
                             f"local {descriptor}, peer {other}")

    def close(self, timeout: float = 0.2) -> None:
        with self._lock:
            if self._closed:
                return
            self._closed = True
            self._stop.set()
            self._wake.set()
            pending = list(self._pending)
            self._pending.clear()
            lanes = list(self._lanes.values())
            self._lanes.clear()
            for lane in lanes:
                lane.queue.put(None)
        self._settle(pending, RuntimeError("point-to-point group was destroyed"))
        self._resolve_queue.put(None)
        end = time.monotonic() + timeout
        for lane in lanes:
            lane.thread.join(max(0.0, end - time.monotonic()))
        self.link.close()


class _Lane:
    def __init__(self, engine: Engine, peer: int, tag: int, sending: bool) -> None:
        self.engine, self.peer, self.tag, self.sending = engine, peer, tag, sending
        self.queue: queue.SimpleQueue = queue.SimpleQueue()
        self.stream: torch.cuda.Stream | None = None
        self.thread = threading.Thread(target=self._loop, name="gpubridge-p2p", daemon=True)
        self.thread.start()

    def _loop(self) -> None:
        while True:
            try:
                item = self.queue.get_nowait()
            except queue.Empty:
                with self.engine._lock:           # the lock submit() queues under
                    if self.queue.empty():
                        key = (self.peer, self.tag, self.sending)
                        if self.engine._lanes.get(key) is self:
                            del self.engine._lanes[key]
                        return
                continue
            if item is None:
                return
            self._one(*item)
            del item

    def _one(self, handle, tensor, ready, deadline, seq) -> None:
        engine = self.engine
        try:
            engine.check()
            stream = None
            if tensor.device.type == "cuda":
                torch.cuda.set_device(tensor.device)
                if self.stream is None or self.stream.device != tensor.device:
                    self.stream = torch.cuda.Stream(tensor.device)
                stream = self.stream
                stream.wait_event(ready)
                tensor.record_stream(stream)
            scope = torch.cuda.stream(stream) if stream is not None else contextlib.nullcontext()
            with scope:
                engine.match(tensor, self.peer, self.tag, seq, self.sending, deadline)
                self._move(tensor, deadline)
                if stream is not None:
                    handle._event = torch.cuda.Event()
                    handle._event.record(stream)
            engine._done(handle)
        except BaseException as exc:  # noqa: BLE001 - delivered through every pending handle
            engine._fail(exc)

    def _left(self, deadline: float) -> timedelta:
        return timedelta(seconds=max(0.001, deadline - time.monotonic()))

    def _move(self, tensor: torch.Tensor, deadline: float) -> None:
        flat = tensor.reshape(-1).view(torch.uint8)     # bytes: any dense dtype travels
        engine = self.engine
        if engine.pinned or engine.chunk_bytes:
            self._chunked(flat, deadline)
            return
        host = flat.cpu() if self.sending else torch.empty(flat.numel(), dtype=torch.uint8)
        engine.link.post(host, self.peer, self.tag, self.sending).wait(self._left(deadline))
        if not self.sending:
            flat.copy_(host)

    def _chunked(self, flat: torch.Tensor, deadline: float) -> None:
        """Two staging slots: a copy overlaps the wire transfer of the other slot."""
        engine = self.engine
        size = engine.chunk_bytes or max(8, flat.numel())
        chunks = list(flat.split(size)) if flat.numel() else [flat]
        staging = make_staging(flat.device, size, min(2, len(chunks)))
        staging.begin(flat)
        try:
            if self.sending:
                staged: dict[int, tuple] = {}

                def stage(i: int) -> None:
                    host = staging.slot(i % 2, chunks[i])
                    staged[i] = (host, staging.to_host(host, chunks[i], None))

                for i in range(min(2, len(chunks))):
                    stage(i)
                for i in range(len(chunks)):
                    host, copied = staged.pop(i)
                    staging.wait_host(copied)
                    engine.link.post(host, self.peer, self.tag, True).wait(self._left(deadline))
                    if i + 2 < len(chunks):
                        stage(i + 2)
            else:
                posted: dict[int, tuple] = {}
                back = [None, None]

                def post(i: int) -> None:
                    staging.wait_host(back[i % 2])
                    host = staging.slot(i % 2, chunks[i])
                    posted[i] = (host, engine.link.post(host, self.peer, self.tag, False))

                for i in range(min(2, len(chunks))):
                    post(i)
                for i, chunk in enumerate(chunks):
                    host, request = posted.pop(i)
                    request.wait(self._left(deadline))
                    back[i % 2] = staging.to_device(chunk, host)
                    if i + 2 < len(chunks):
                        post(i + 2)
                staging.end(back[(len(chunks) - 1) % 2])
        finally:
            staging.close()
