"""Async collectives: the :class:`Work` handle and the two ways a collective is started.

* **Queued** (host-staged policies, CPU simulation): one worker thread per rank with its
  own CUDA stream runs queued collectives first in, first out, exactly like the reference
  (src/gpubridge/work.py:118-205): an event recorded on the caller's stream gates the
  worker stream, tensors are ``record_stream``-ed, ``Work.wait`` blocks the host until the
  worker ran the call and then orders the caller's stream after the worker's event.  The
  queue is bounded (``GPUBRIDGE_ASYNC_QUEUE``, default 1024); the first failure poisons the
  rank: every later collective refuses to start.
* **Stream-ordered** (fused NVLink kernels): the launch is non-blocking, so it happens on
  the calling thread onto the fabric's communication stream, ordered by events both ways.
  ``Work.wait`` then never blocks the host, which is the NCCL behaviour the reference
  documents it lacks (docs/TORCH_BACKEND.md:165-167).  FIFO order with queued work is kept
  by draining the queue first.
"""
from __future__ import annotations

import os
import queue
import threading
from collections.abc import Callable, Sequence
from datetime import timedelta
from typing import Any

import torch

from gpubridge_b200._mutation import mutated

QUEUE_ENV = "GPUBRIDGE_ASYNC_QUEUE"
DEFAULT_QUEUE = 1024


def queue_limit() -> int:
    raw = os.environ.get(QUEUE_ENV, "").strip()
    try:
        limit = int(raw) if raw else DEFAULT_QUEUE
    except ValueError:
        limit = 0
    if limit <= 0:
        raise ValueError(f"{QUEUE_ENV} must be a positive whole number")
    return limit


class Work:
    """Handle of one async collective; mirrors ``torch.distributed.Work``."""

    def __init__(self, op: str, device: torch.device, result: Any) -> None:
        self.op = op
        self._device = device
        self._result = result
        self._done = threading.Event()
        self._error: BaseException | None = None
        self._event: torch.cuda.Event | None = None
        self._check: Callable[[], None] | None = None   # raises if the device reported a failure
        self._future: torch.futures.Future = torch.futures.Future(
            devices=[device] if device.type == "cuda" else [])

    def is_completed(self) -> bool:
        """True once the collective ended on this rank, device work included.  Never blocks."""
        if not self._done.is_set():
            return False
        return self._event is None or self._event.query()

    def wait(self, timeout: timedelta | float | None = None) -> bool:
        seconds = timeout.total_seconds() if isinstance(timeout, timedelta) else timeout
        if not self._done.wait(seconds):
            raise TimeoutError(f"gpubridge async {self.op} did not finish within {seconds} s")
        if self._error is not None:
            raise RuntimeError(f"gpubridge async {self.op} failed: {self._error}") from self._error
        if self._event is not None and not mutated("wait-skips-stream"):
            torch.cuda.current_stream(self._device).wait_event(self._event)
        if self._check is not None and self._event is not None and self._event.query():
            self._check()
        return True

    def exception(self) -> BaseException | None:
        return self._error

    def get_future(self) -> torch.futures.Future:
        """Holds the output tensor (None for a barrier) once the collective ends."""
        return self._future

    def _finish(self, error: BaseException | None) -> None:
        self._error = error
        if error is None:
            self._future.set_result(self._result)
        else:
            self._future.set_exception(error)
        self._done.set()


class _Worker:
    def __init__(self, device: torch.device) -> None:
        self.device = device
        self.limit = queue_limit()
        # a SimpleQueue (one C-level lock) plus a count of accepted items: cheaper per call
        # than queue.Queue's two condition variables, with the same bound and join()
        self.queue: queue.SimpleQueue = queue.SimpleQueue()
        self._accepted = 0
        self._count_lock = threading.Lock()
        self._idle = threading.Event()
        self._idle.set()
        self.failed: BaseException | None = None
        self.stream: torch.cuda.Stream | None = None
        self.thread = threading.Thread(target=self._loop, name="gpubridge-async", daemon=True)
        self.thread.start()

    def submit(self, op, fn, tensors, result) -> Work:
        work = Work(op, self.device, result)
        ready = None
        if self.device.type == "cuda":
            ready = torch.cuda.Event()
            ready.record(torch.cuda.current_stream(self.device))
        with self._count_lock:
            if self._accepted >= self.limit:
                raise RuntimeError(
                    f"gpubridge async queue is full ({self.limit} queued collectives); wait for "
                    "accepted work before retrying this collective, preserving the same "
                    f"collective order on every rank ({QUEUE_ENV})")
            self._accepted += 1
            self._idle.clear()
        self.queue.put((work, fn, ready, tuple(tensors)))
        return work

    def _retire(self) -> None:
        with self._count_lock:
            self._accepted -= 1
            if self._accepted == 0:
                self._idle.set()

    def join(self) -> None:
        """Until everything accepted so far has run."""
        self._idle.wait()

    def _loop(self) -> None:
        if self.device.type == "cuda":
            torch.cuda.set_device(self.device)
            self.stream = torch.cuda.Stream(self.device)
        while True:
            item = self.queue.get()
            try:
                if item is None:
                    return
                work, fn, ready, tensors = item
                if self.failed is not None:
                    work._finish(RuntimeError("not run: an earlier async collective failed on "
                                              f"this rank ({self.failed})"))
                    continue
                try:
                    self._one(work, fn, ready, tensors)
                except BaseException as error:  # noqa: BLE001 - carried by the Work
                    self.failed = error
                    work._finish(error)
            finally:
                if item is not None:
                    self._retire()

    def _one(self, work, fn, ready, tensors) -> None:
        if self.stream is None:
            fn()
            work._finish(None)
            return
        self.stream.wait_event(ready)
        for t in tensors:
            t.record_stream(self.stream)
        with torch.cuda.stream(self.stream):
            fn()
            work._event = torch.cuda.Event()
            work._event.record(self.stream)
            work._finish(None)

    def close(self) -> None:
        self.queue.put(None)
        self.thread.join()

    def abandon(self, timeout: float) -> None:
        while True:
            try:
                item = self.queue.get_nowait()
            except queue.Empty:
                break
            if item is not None:
                item[0]._finish(RuntimeError(f"gpubridge async {item[0].op} not run: its "
                                             "process groups were destroyed"))
                self._retire()
        self.queue.put(None)
        self.thread.join(timeout)


_worker: _Worker | None = None
_poison: BaseException | None = None


def poison(error: BaseException) -> None:
    """Record a failure seen outside the worker (a device-side wait that ran out)."""
    global _poison
    if _poison is None:
        _poison = error


def check_healthy() -> None:
    failed = _poison or (_worker.failed if _worker is not None else None)
    if failed is not None:
        raise RuntimeError(
            f"an earlier async gpubridge collective failed on this rank ({type(failed).__name__}: "
            f"{failed}); the process groups may be inconsistent. Call gpubridge.destroy() and "
            "init() again (under the torch.distributed backend: destroy_process_group() and "
            "init_process_group()).")


def submit(device: torch.device, op: str, fn: Callable[[], None],
           tensors: Sequence[torch.Tensor], result: Any) -> Work:
    """Queue ``fn`` on the worker thread (started at first use)."""
    global _worker
    check_healthy()
    if _worker is None:
        _worker = _Worker(device)
    return _worker.submit(op, fn, tensors, result)


def launch(device: torch.device, op: str, fn: Callable[[], "torch.cuda.Event | None"],
           result: Any, check: Callable[[], None] | None = None,
           stream: "torch.cuda.Stream | None" = None) -> Work:
    """Start a stream-ordered collective now, on the calling thread.  ``fn`` enqueues the
    device work on ``stream`` and returns the event recorded after it."""
    check_healthy()
    if _worker is not None:
        _worker.join()            # keep program order with queued collectives
        check_healthy()
    work = Work(op, device, result)
    try:
        work._event = fn()
        work._check = check
    except BaseException as error:  # noqa: BLE001
        poison(error)
        work._finish(error)
        raise
    if stream is not None:
        with torch.cuda.stream(stream):   # the device-aware future records on this stream
            work._finish(None)
    else:
        work._finish(None)
    return work


def drain() -> None:
    if _worker is not None:
        _worker.join()
    check_healthy()


def shutdown() -> None:
    """Run what is queued, stop the worker, forget failures (init/destroy call this)."""
    global _worker, _poison
    worker, _worker = _worker, None
    _poison = None
    if worker is not None:
        worker.close()


def abandon(timeout: float = 10.0) -> None:
    """Stop the worker without running what is queued: each queued collective fails."""
    global _worker, _poison
    worker, _worker = _worker, None
    _poison = None
    if worker is not None:
        worker.abandon(timeout)
