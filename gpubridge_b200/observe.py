"""Watching collectives: observers, per-phase timing and the in-flight table.

Same contract as the reference (src/gpubridge/observe.py:55-450): every collective takes a
sequence number that is equal on all ranks; an observer gets a :class:`CollectiveRecord`
right after the call, on the thread that ran it; time marks are CUDA timing events on the
current stream (never a device synchronisation) and exist only while somebody watches;
:func:`in_flight` is a lock-free host view for watchdogs; an observer may not communicate
and one that raises is detached with a warning.

B200 addition: a fused kernel reports its internal steps as device timestamps
(``globaltimer`` values), which :func:`device_phases` turns into ordinary phases, so an
observer sees "island-reduce / bridge / island-broadcast" although one launch ran them.
"""
from __future__ import annotations

import abc
import os
import threading
import time
import warnings
from dataclasses import dataclass, field
from typing import TYPE_CHECKING

import torch

if TYPE_CHECKING:
    from gpubridge_b200.topology import Topology


@dataclass(frozen=True)
class Mark:
    """A point in time: when the host reached it and, on GPUs, when the stream did."""

    host_ns: int
    event: "torch.cuda.Event | None" = None
    device_ns: int | None = None
    """A ``globaltimer`` reading taken inside a kernel; set for phases of fused kernels."""
    source: "tuple[torch.Tensor, int] | None" = None
    """Where a ``globaltimer`` reading will be once ``event`` has completed: element ``i`` of
    a pinned host tensor that an asynchronous copy fills (no host wait when the mark is made)."""

    def ready(self) -> bool:
        return self.event is None or self.event.query()

    def ns(self) -> int | None:
        """The device timestamp, if this mark has one (read it only when :meth:`ready`)."""
        if self.device_ns is not None:
            return self.device_ns
        if self.source is not None:
            return int(self.source[0][self.source[1]])
        return None


def elapsed_ms(start: Mark, end: Mark) -> float:
    """Milliseconds between two ready marks, on the device clock when both have one."""
    a, b = start.ns(), end.ns()
    if a is not None and b is not None:
        return (b - a) / 1e6
    if start.event is not None and end.event is not None:
        return start.event.elapsed_time(end.event)
    return (end.host_ns - start.host_ns) / 1e6


@dataclass(frozen=True)
class Phase:
    name: str
    start: Mark
    end: Mark

    def elapsed_ms(self) -> float:
        return elapsed_ms(self.start, self.end)


@dataclass(frozen=True)
class CollectiveRecord:
    """One collective on this rank."""

    seq: int
    op: str
    nbytes: int
    dtype: torch.dtype | None
    src: int | None
    policy: str | None
    start: Mark
    end: Mark
    phases: tuple[Phase, ...] = ()
    reduce_op: str | None = None

    def ready(self) -> bool:
        marks = [self.start, self.end, *(m for p in self.phases for m in (p.start, p.end))]
        return all(m.ready() for m in marks)

    def elapsed_ms(self) -> float:
        return elapsed_ms(self.start, self.end)

    def phase(self, name: str) -> Phase | None:
        for p in self.phases:
            if p.name == name:
                return p
        return None


class CollectiveObserver(abc.ABC):
    """Receives every collective's record.  Keep ``on_collective`` cheap; never communicate."""

    @abc.abstractmethod
    def on_collective(self, record: CollectiveRecord) -> None: ...

    def on_detach(self, error: BaseException) -> None:  # noqa: B027 - optional
        """Called once when the observer is dropped because ``on_collective`` raised."""


@dataclass(frozen=True)
class InFlight:
    """A collective some thread of this rank is inside right now."""

    seq: int
    op: str
    policy: str | None
    phase: str | None
    phases_done: tuple[str, ...]
    thread: str
    seconds: float


@dataclass
class _Flight:
    seq: int
    op: str
    policy: str | None
    phase: str | None = None
    done: tuple[str, ...] = ()
    ident: int = 0
    since: float = 0.0
    phases: list[Phase] = field(default_factory=list)
    device: torch.device | None = None   # set when somebody is watching: time with events
    watched: bool = False


class _Local(threading.local):
    flight: _Flight | None = None
    in_callback: bool = False


_local = _Local()
_observers: list[CollectiveObserver] = []
_table: dict[int, _Flight] = {}
_seq = 0
_seq_lock = threading.Lock()


def add_observer(observer: CollectiveObserver) -> None:
    from gpubridge_b200.topology import get_topology
    get_topology()  # raises when not initialised
    if not isinstance(observer, CollectiveObserver):
        raise TypeError(f"expected a CollectiveObserver, got {type(observer).__name__}")
    if observer not in _observers:
        _observers.append(observer)


def remove_observer(observer: CollectiveObserver) -> None:
    if observer in _observers:
        _observers.remove(observer)


def watching() -> bool:
    return bool(_observers)


def in_flight() -> list[InFlight]:
    """Oldest first; never blocks, communicates or touches a device."""
    flights: list[_Flight] = []
    for _ in range(10):
        try:
            flights = list(_table.values())
            break
        except RuntimeError:  # resized while copying
            continue
    now = time.monotonic()
    names = {t.ident: t.name for t in threading.enumerate()}
    rows = [InFlight(f.seq, f.op, f.policy, f.phase, f.done, names.get(f.ident, str(f.ident)),
                     now - f.since) for f in flights if f.ident]
    return sorted(rows, key=lambda r: r.seq)


def _reset() -> None:
    global _seq
    _observers.clear()
    _table.clear()
    with _seq_lock:
        _seq = 0
    _local.flight = None
    _local.in_callback = False


def refuse_in_callback(op: str) -> None:
    if _local.in_callback:
        raise RuntimeError(f"gpubridge.{op}() called from inside a collective observer; "
                           "observers must not communicate")


def _mark(device: torch.device | None) -> Mark:
    if device is None:
        return Mark(time.perf_counter_ns())
    event = torch.cuda.Event(enable_timing=True)
    event.record(torch.cuda.current_stream(device))
    return Mark(time.perf_counter_ns(), event)


def _nvtx_setting():
    """``torch.cuda.nvtx`` when ``GPUBRIDGE_NVTX=1`` and the build has it, else None.  Ranges
    named ``gpubridge.<op> <bytes>`` (and ``gpubridge.<phase>`` inside them) then show every
    collective on the host timeline of a profiler that reads NVTX."""
    if os.environ.get("GPUBRIDGE_NVTX", "0") != "1":
        return None
    try:
        from torch.cuda import nvtx
        nvtx.range_push("gpubridge.nvtx-check")
        nvtx.range_pop()
        return nvtx
    except Exception:  # noqa: BLE001 - a build without NVTX: ranges are an extra, never an error
        return None


_nvtx = _nvtx_setting()


def reload_nvtx() -> bool:
    """Read ``GPUBRIDGE_NVTX`` again (it is read once, at import); True when ranges are on."""
    global _nvtx
    _nvtx = _nvtx_setting()
    return _nvtx is not None


class collective:  # noqa: N801 - used as ``with collective(...)``
    """Count one validated collective, list it as in flight, record it if watched."""

    def __init__(self, topology: "Topology", op: str, tensor: torch.Tensor | None = None, *,
                 src: int | None = None, policy: str | None = None,
                 reduce_op: str | None = None) -> None:
        global _seq
        refuse_in_callback(op)
        with _seq_lock:
            seq, _seq = _seq, _seq + 1
        self.flight = _Flight(seq, op, policy)
        self.flight.watched = bool(_observers)
        if self.flight.watched and topology.device.type == "cuda":
            self.flight.device = topology.device
        self.tensor, self.src, self.reduce_op = tensor, src, reduce_op

    def __enter__(self) -> None:
        f = self.flight
        f.ident, f.since = threading.get_ident(), time.monotonic()
        _table[f.ident] = f
        _local.flight = f
        if _nvtx is not None:
            _nvtx.range_push(f"gpubridge.{f.op} {0 if self.tensor is None else self.tensor.nbytes}")
        if f.watched:
            self.start = _mark(f.device)

    def __exit__(self, exc_type, *exc) -> None:
        f = self.flight
        _table.pop(f.ident, None)
        _local.flight = None
        if _nvtx is not None:
            _nvtx.range_pop()
        if exc_type is not None or not f.watched:
            return
        t = self.tensor
        _deliver(CollectiveRecord(
            seq=f.seq, op=f.op, nbytes=0 if t is None else t.nbytes,
            dtype=None if t is None else t.dtype, src=self.src, policy=f.policy,
            start=self.start, end=_mark(f.device), phases=tuple(f.phases),
            reduce_op=self.reduce_op))


class _NoPhase:
    def __enter__(self): return None
    def __exit__(self, *exc): return None


_NO_PHASE = _NoPhase()


class _PhaseScope:
    def __init__(self, flight: _Flight, name: str) -> None:
        self.flight, self.name = flight, name

    def __enter__(self) -> None:
        f = self.flight
        self.outer, f.phase = f.phase, self.name
        if _nvtx is not None:
            _nvtx.range_push(f"gpubridge.{self.name}")
        if f.watched:
            self.start = _mark(f.device)

    def __exit__(self, exc_type, *exc) -> None:
        f = self.flight
        f.phase = self.outer
        if _nvtx is not None:
            _nvtx.range_pop()
        f.done = (*f.done, self.name)
        if exc_type is None and f.watched:
            f.phases.append(Phase(self.name, self.start, _mark(f.device)))


def phase(name: str):
    """Mark one step of the collective the calling thread is inside (no-op outside one)."""
    flight = _local.flight
    return _NO_PHASE if flight is None else _PhaseScope(flight, name)


def device_phases(names: list[str], stamps_ns: list[int]) -> None:
    """Attach phases measured inside a fused kernel: ``stamps_ns`` holds ``len(names)+1``
    ``globaltimer`` readings, phase i running from stamp i to stamp i+1."""
    flight = _local.flight
    if flight is None:
        return
    flight.done = (*flight.done, *names)
    if not flight.watched:
        return
    host = time.perf_counter_ns()
    for i, name in enumerate(names):
        flight.phases.append(Phase(name, Mark(host, None, stamps_ns[i]),
                                   Mark(host, None, stamps_ns[i + 1])))


def device_phases_later(names: list[str], stamps: torch.Tensor, event) -> None:
    """Like :func:`device_phases` for timestamps that an asynchronous copy is still bringing to
    ``stamps`` (pinned host memory, ``len(names) + 1`` values); ``event`` completes after the
    copy.  The phases are ready when the event is."""
    flight = _local.flight
    if flight is None:
        return
    flight.done = (*flight.done, *names)
    if not flight.watched:
        return
    host = time.perf_counter_ns()
    for i, name in enumerate(names):
        flight.phases.append(Phase(name, Mark(host, event, None, (stamps, i)),
                                   Mark(host, event, None, (stamps, i + 1))))


def _deliver(record: CollectiveRecord) -> None:
    for observer in tuple(_observers):
        _local.in_callback = True
        try:
            observer.on_collective(record)
        except Exception as error:  # noqa: BLE001 - any failure detaches the observer
            remove_observer(observer)
            warnings.warn(f"gpubridge detached collective observer {observer!r} on this rank "
                          f"after it raised {type(error).__name__}: {error}. Collectives "
                          "continue without it.", RuntimeWarning, stacklevel=4)
            try:
                observer.on_detach(error)
            except Exception:  # noqa: BLE001, S110
                pass
        finally:
            _local.in_callback = False
