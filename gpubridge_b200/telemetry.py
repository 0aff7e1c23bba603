"""Observations as JSON lines: what a long run leaves behind for later analysis.

    emitter = Emitter(path, run="fsdp2-1.3b", rank=rank)
    emitter.emit("collective", op="all_reduce", nbytes=1 << 20, ms=0.21)
    emitter.endpoint(endpoint)          # an rdma endpoint's counters, as one record
    emitter.close()

One JSON object per line, each with ``time`` (seconds since the epoch), ``kind``, and the run's
constant fields.  Writing happens on a daemon thread behind a bounded queue, so ``emit`` costs a
dictionary and a queue put and never blocks the training loop: when the queue is full the
record is dropped and counted (``dropped`` is written with the next record that gets through,
and at close).  Records go to ``PATH.partial`` and the file takes its name at ``close()``, so a
reader never sees half a run mistaken for a whole one.

Field names that look like credentials or remote-memory keys are refused (``ValueError``), so a
record can be shared without a review: names containing ``key``, ``secret``, ``token``,
``password`` or ``credential`` (reference: src/gpubridge/verbs/observe.py:39-63, 125-199 - its
emitter for the verbs bridge; this one serves every part of the library).  An
:class:`~gpubridge_b200.observe.CollectiveObserver` that emits every collective is included.
"""
from __future__ import annotations

import json
import os
import queue
import threading
import time
from typing import Any

from gpubridge_b200 import observe as _observe

FORBIDDEN = ("key", "secret", "token", "password", "credential")
PLAIN = (str, int, float, bool, type(None))


def check_fields(fields: dict[str, Any]) -> None:
    """Raise ``ValueError`` for a field whose name suggests a secret or whose value is not a plain
    JSON scalar, list or dict of such."""
    for name, value in fields.items():
        lowered = name.lower()
        if any(word in lowered for word in FORBIDDEN):
            raise ValueError(f"telemetry field {name!r} looks like a credential or a memory key; "
                             "records must be shareable as they are")
        _check_value(name, value)


def _check_value(name: str, value: Any) -> None:
    if isinstance(value, PLAIN):
        return
    if isinstance(value, (list, tuple)):
        for item in value:
            _check_value(name, item)
        return
    if isinstance(value, dict):
        check_fields(value)
        return
    raise ValueError(f"telemetry field {name!r} holds a {type(value).__name__}; only JSON values travel")


class Emitter:
    """Writes records to ``path`` as JSON lines from a background thread."""

    def __init__(self, path: str | os.PathLike, *, capacity: int = 4096, **constant: Any) -> None:
        check_fields(constant)
        self.path = os.fspath(path)
        self.constant = dict(constant)
        self.dropped = self.written = 0
        self._queue: queue.Queue = queue.Queue(maxsize=capacity)
        self._closed = False
        os.makedirs(os.path.dirname(os.path.abspath(self.path)) or ".", exist_ok=True)
        self._file = open(self.path + ".partial", "w", buffering=1)
        self._thread = threading.Thread(target=self._write, name="gpubridge-telemetry", daemon=True)
        self._thread.start()

    def emit(self, kind: str, **fields: Any) -> bool:
        """Queue one record; False when it was dropped (queue full or emitter closed)."""
        check_fields(fields)
        if self._closed:
            return False
        record = {"time": round(time.time(), 6), "kind": kind, **self.constant, **fields}
        try:
            self._queue.put_nowait(record)
            return True
        except queue.Full:
            self.dropped += 1
            return False

    def endpoint(self, endpoint) -> bool:
        """The counters of an :class:`gpubridge_b200.rdma.Endpoint` as one ``endpoint`` record."""
        return self.emit("endpoint", **endpoint.telemetry())

    def _write(self) -> None:
        reported = 0
        while True:
            record = self._queue.get()
            if record is None:
                break
            if self.dropped != reported:
                record["dropped_before"] = reported = self.dropped
            self._file.write(json.dumps(record, separators=(",", ":")) + "\n")
            self.written += 1
        self._file.write(json.dumps({"time": round(time.time(), 6), "kind": "closed", **self.constant,
                                     "written": self.written, "dropped": self.dropped}) + "\n")

    def close(self) -> None:
        """Write what is queued, add a closing record with the totals, give the file its name."""
        if self._closed:
            return
        self._closed = True
        self._queue.put(None)
        self._thread.join(10)
        self._file.close()
        os.replace(self.path + ".partial", self.path)

    def __enter__(self) -> "Emitter":
        return self

    def __exit__(self, *exc) -> None:
        self.close()


class CollectiveEmitter(_observe.CollectiveObserver):
    """``add_observer(CollectiveEmitter(emitter))``: one ``collective`` record per collective,
    with its phases once their timings are known."""

    def __init__(self, emitter: Emitter) -> None:
        self.emitter = emitter

    def on_collective(self, record) -> None:
        phases = {p.name: round(p.elapsed_ms(), 4) for p in record.phases
                  if p.start.ready() and p.end.ready()}
        ms = round(record.elapsed_ms(), 4) if record.ready() else None
        self.emitter.emit("collective", seq=record.seq, op=record.op, nbytes=record.nbytes,
                          dtype=str(record.dtype) if record.dtype is not None else None,
                          policy=record.policy, reduce_op=record.reduce_op, ms=ms, phases=phases)
