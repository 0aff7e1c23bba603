"""Bridge transports whose collectives run inside a native tagged-message worker.

A *worker* (today: the multi-stream TCP worker of ``csrc/gb_tcp.cpp``) owns the connections
between the bridge members and implements ``all_reduce`` and ``broadcast`` itself, chunked and
pipelined, without a Python round trip per message.  What is left for Python is the part that
involves the job's store - agreeing that the link is up, on every rank - and guarding the
worker's lifetime.  This file is that part; a transport subclass only supplies
:meth:`TaggedBridge._connect`.

Behaviour a user of the reference relies on (src/gpubridge/tagged.py) and that holds here:

* **Everyone learns the outcome of link setup.**  Each member publishes ``ok`` or its error
  under a status key; members and non-members alike read all of them and raise the same
  message if any member failed, so no rank waits forever for a bridge that never came up.
* **A first message proves the link.**  Before a transport is handed out, its members run one
  tiny all-reduce through the worker; wiring mistakes fail here, not in step 1000.
* **Nothing outlives the tensors.**  If a collective raises, the worker is aborted first, so
  no posted receive can write into memory the caller has already released.
* **Reduction order is fixed**: two members add the peer's values to their own; more members
  run a ring whose segment *j* starts at member *j* and walks upward (:func:`ring_order`),
  and ``segments`` says where the segments lie.  Tests rebuild the expected bits from these
  two functions alone.
"""
from __future__ import annotations

import contextlib
import time
from collections.abc import Iterator, Sequence
from datetime import timedelta
from typing import Any, ClassVar

import torch

from gpubridge_b200.transport import BridgeTransport, LinkContext

DEFAULT_TIMEOUT = timedelta(minutes=30)

#: element-type and operation codes of the native collectives (csrc/gb_tcp.cpp)
DTYPE_CODES = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2, torch.float64: 3,
               torch.int8: 4, torch.uint8: 5, torch.int32: 6, torch.int64: 7}
OP_CODES = {"sum": 0, "max": 1, "min": 2}


def segments(numel: int, parts: int) -> list[tuple[int, int]]:
    """Where the ring cuts a tensor: ``parts`` consecutive (start, length) pieces of near-equal
    size, the remainder spread one element each over the leading pieces."""
    quotient, remainder = divmod(numel, parts)
    lengths = [quotient + (index < remainder) for index in range(parts)]
    starts = [sum(lengths[:index]) for index in range(parts)]
    return list(zip(starts, lengths))


def ring_order(segment: int, members: int) -> list[int]:
    """The members in the order their values enter the sum of ``segment``: the member with the
    segment's own index first, then upward around the ring."""
    return [(segment + hop) % members for hop in range(members)]


class Guarded:
    """Lifetime of a native worker's handle when several threads use it.

    Every call into the library goes through :meth:`_inside`, which counts the calls that are
    in there; :meth:`_retire` (from ``close``) refuses new calls, asks the library to end the
    ones inside (``stop``: the native abort, after which their waits return with an error),
    waits - for a bounded time - until they have left, and only then hands the handle to
    ``free``.  A call on a closed worker raises instead of handing the library nothing.
    """

    _what = "worker"

    def _guard(self) -> None:
        import threading
        self._gate = threading.Condition()
        self._calls_inside = 0
        self._closing = False

    @contextlib.contextmanager
    def _inside(self):
        with self._gate:
            if self._closing or not getattr(self, "handle", None):
                raise RuntimeError(f"{self._what}: the worker is closed")
            self._calls_inside += 1
        try:
            yield self.handle
        finally:
            with self._gate:
                self._calls_inside -= 1
                self._gate.notify_all()

    def _retire(self, stop, free, limit: float = 10.0) -> bool:
        """True when the handle was freed now; False when it was closed before or calls were
        still inside at the limit (the handle is then leaked rather than freed under them)."""
        with self._gate:
            if self._closing or not getattr(self, "handle", None):
                return False
            self._closing = True
            handle = self.handle
            if self._calls_inside:
                stop(handle)
                if not self._gate.wait_for(lambda: self._calls_inside == 0, limit):
                    self.handle = None
                    return False
            self.handle = None
        free(handle)
        return True


def message_tag(number: int, step: int, sender: int, chunk: int) -> int:
    """The 64-bit tag of one message, as the native collectives number them: call (24 bits),
    step (12), sending member (8), chunk (20)."""
    return ((number & 0xFFFFFF) << 40) | ((step & 0xFFF) << 28) | ((sender & 0xFF) << 20) | (chunk & 0xFFFFF)


_FOLDS = {"sum": lambda mine, theirs: mine.add_(theirs),
          "max": lambda mine, theirs: torch.maximum(mine, theirs, out=mine),
          "min": lambda mine, theirs: torch.minimum(mine, theirs, out=mine)}


class OnDevice:
    """The collectives of the native workers, message by message from Python, for tensors whose
    reduction has to run where they live: a worker that reads and writes device memory itself
    (GPUDirect) cannot fold on the host.  Same cuts, order and tags as ``csrc/gb_tagged.cpp``;
    the worker only needs ``send(peer, pointer, nbytes, tag)``, ``recv(...)`` and
    ``wait(ids, deadline)``.

    ``settle`` runs before messages are posted (the producer of the bytes must have finished:
    a stream synchronise for device tensors) and ``landed`` after receives completed and before
    anything reads them (the flush of direct writes, where the device needs one).
    """

    def __init__(self, worker: Any, members: int, index: int, settle=None, landed=None) -> None:
        self.worker, self.members, self.index = worker, members, index
        self.settle = settle or (lambda: None)
        self.landed = landed or (lambda: None)

    def _post(self, sending: bool, peer: int, flat: torch.Tensor, chunk: int, number: int, step: int,
              sender: int, ids: list[int]) -> None:
        esize, base, count = flat.element_size(), flat.data_ptr(), flat.numel()
        starts = range(0, count, chunk) if count else [0]
        for index, start in enumerate(starts):
            n = min(chunk, count - start)
            call = self.worker.send if sending else self.worker.recv
            ids.append(call(peer, base + start * esize, n * esize, message_tag(number, step, sender, index)))

    def all_reduce(self, flat: torch.Tensor, op: str, chunk_elems: int, number: int, deadline: float) -> None:
        size, me, fold = self.members, self.index, _FOLDS[op]
        if size == 1 or flat.numel() == 0:
            return
        chunk = max(1, chunk_elems)
        if size == 2:
            scratch = torch.empty_like(flat)
            ids: list[int] = []
            self.settle()
            self._post(False, 1 - me, scratch, chunk, number, 0, 1 - me, ids)
            self._post(True, 1 - me, flat, chunk, number, 0, me, ids)
            self.worker.wait(ids, deadline)
            self.landed()
            fold(flat, scratch)
            return
        cuts = segments(flat.numel(), size)
        piece = lambda i: flat.narrow(0, *cuts[i % size])                      # noqa: E731
        scratch = torch.empty(cuts[0][1], dtype=flat.dtype, device=flat.device)
        right, left = (me + 1) % size, (me - 1) % size
        for step in range(size - 1):                                           # reduce-scatter
            arriving, leaving = piece(me - step - 1), piece(me - step)
            ids = []
            self.settle()
            self._post(False, left, scratch[:arriving.numel()], chunk, number, step, left, ids)
            self._post(True, right, leaving, chunk, number, step, me, ids)
            self.worker.wait(ids, deadline)
            self.landed()
            fold(arriving, scratch[:arriving.numel()])
        for step in range(size - 1):                                           # all-gather
            ids = []
            self.settle()
            self._post(False, left, piece(me - step), chunk, number, size + step, left, ids)
            self._post(True, right, piece(me + 1 - step), chunk, number, size + step, me, ids)
            self.worker.wait(ids, deadline)
        self.landed()

    def broadcast(self, flat: torch.Tensor, root: int, chunk_bytes: int, number: int, deadline: float) -> None:
        if self.members == 1 or flat.numel() == 0:
            return
        raw = flat.view(torch.uint8)
        ids: list[int] = []
        self.settle()
        if self.index == root:
            for peer in range(self.members):
                if peer != root:
                    self._post(True, peer, raw, max(1, chunk_bytes), number, 0, root, ids)
        else:
            self._post(False, root, raw, max(1, chunk_bytes), number, 0, root, ids)
        self.worker.wait(ids, deadline)
        if self.index != root:
            self.landed()


def wait_for_keys(store, keys: Sequence[str], deadline: float, what: str,
                  verdicts: Sequence[str] = ()) -> list[str]:
    """Values of ``keys`` once all exist; polls in short slices so the deadline is honoured
    whatever timeout type the store raises.  ``verdicts`` are keys under which members publish
    how their set-up ended: as soon as one of them holds anything but ``ok`` the wait is over -
    that member will never publish what is waited for."""
    wanted = list(keys)
    while True:
        slice_s = max(0.05, min(0.5 if verdicts else 2.0, deadline - time.monotonic()))
        try:
            store.wait(wanted, timedelta(seconds=slice_s))
        except Exception:  # noqa: BLE001
            for key in verdicts:
                try:
                    store.wait([key], timedelta(milliseconds=1))
                    said = store.get(key).decode()
                except Exception:  # noqa: BLE001 - not published yet
                    continue
                if said != "ok":
                    raise RuntimeError(f"gave up waiting for {what}: another member's set-up failed") from None
            if time.monotonic() >= deadline:
                raise RuntimeError(f"timed out waiting for {what}") from None
            continue
        return [store.get(key).decode() for key in wanted]


class TaggedBridge(BridgeTransport):
    """A bridge over a native worker.  Subclasses set ``name`` and implement :meth:`_connect`,
    which returns an instance whose worker is connected to every other member."""

    reduce_ops = frozenset(OP_CODES)
    _instead: ClassVar[str] = 'use bridge="gloo" to run without it'

    def __init__(self, worker: Any, members: Sequence[int], rank: int, timeout: timedelta,
                 chunk_bytes: int) -> None:
        self.worker = worker
        self.members = list(members)
        self.index = self.members.index(rank)
        self.timeout = timeout.total_seconds()
        self.chunk_bytes = chunk_bytes
        self._calls = 0                      # the sequence number that keeps calls' messages apart

    # -- setup: collective over ALL ranks of the job ----------------------------------------------
    @classmethod
    def create(cls, ranks, *, context: LinkContext, timeout=None):
        timeout = timeout or DEFAULT_TIMEOUT
        members = list(ranks)
        base = f"gb/{cls.name}/{context.name}/{'_'.join(str(m) for m in members)}"
        deadline = time.monotonic() + timeout.total_seconds()
        transport = None
        if context.rank in members:
            verdict = "ok"
            try:
                transport = cls._connect(context.store, base, members, context.rank, timeout, deadline)
                transport.prove(deadline)
            except Exception as failure:  # noqa: BLE001 - becomes every rank's error below
                verdict = f"{type(failure).__name__}: {failure}"
                if transport is not None:
                    transport.close()
                    transport = None
            context.store.set(f"{base}/status/{context.rank}", verdict)
        verdicts = wait_for_keys(context.store, [f"{base}/status/{m}" for m in members], deadline,
                                 f"every bridge member to report on its {cls.name} connections")
        broken = {m: v for m, v in zip(members, verdicts) if v != "ok"}
        if not broken:
            return transport
        if transport is not None:
            transport.close()
        lines = "\n".join(f"  rank {m}: {v}" for m, v in broken.items())
        raise RuntimeError(f"The {cls.name} bridge between ranks {members} could not be set up; "
                           f"{cls._instead}.\n{lines}")

    @classmethod
    def _connect(cls, store, key, members, rank, timeout, deadline) -> "TaggedBridge":
        raise NotImplementedError

    @classmethod
    def create_p2p(cls, group, *, store=None, timeout=None):
        """Cross-island point-to-point of a bridge without a wire of its own for it: the job's
        Gloo group carries the engine's host buffers (a subclass may bring its own link)."""
        from gpubridge_b200.p2p import GlooLink
        return GlooLink(group)

    def prove(self, deadline: float) -> None:
        """One all-reduce of the members' indices: the sum is known in advance."""
        count = len(self.members)
        if count == 1:
            return
        probe = torch.tensor([self.index], dtype=torch.int64)
        self._calls += 1
        self.worker.all_reduce(probe.data_ptr(), 1, DTYPE_CODES[torch.int64], OP_CODES["sum"], 1,
                               self._calls, deadline)
        if int(probe) != count * (count - 1) // 2:
            raise RuntimeError(f"the {self.name} link came up but its first sum was {int(probe)}, "
                               f"not {count * (count - 1) // 2}: members are wired to the wrong peers")

    # -- collectives ---------------------------------------------------------------------------------
    @contextlib.contextmanager
    def _call(self, tensor: torch.Tensor) -> Iterator[tuple[int, float]]:
        """Validate, number the call, and make sure a failure stops the worker before it
        reaches the caller."""
        if tensor.device.type != "cpu" or not tensor.is_contiguous():
            raise ValueError(f"the {self.name} bridge carries contiguous host tensors")
        if tensor.dtype not in DTYPE_CODES:
            raise ValueError(f"the {self.name} bridge cannot carry {tensor.dtype}")
        self._calls += 1
        try:
            yield self._calls, time.monotonic() + self.timeout
        except BaseException:
            self.worker.abort()
            raise

    def all_reduce(self, tensor: torch.Tensor, op: str = "sum") -> None:
        if len(self.members) == 1 or tensor.numel() == 0:
            return
        with self._call(tensor) as (number, deadline):
            per_chunk = max(1, self.chunk_bytes // tensor.element_size())
            self.worker.all_reduce(tensor.data_ptr(), tensor.numel(), DTYPE_CODES[tensor.dtype],
                                   OP_CODES[op], per_chunk, number, deadline)

    def broadcast(self, tensor: torch.Tensor, src: int) -> None:
        if len(self.members) == 1 or tensor.numel() == 0:
            return
        with self._call(tensor) as (number, deadline):
            self.worker.broadcast(tensor.data_ptr(), tensor.numel() * tensor.element_size(),
                                  self.members.index(src), max(1, self.chunk_bytes), number, deadline)

    def close(self) -> None:
        worker, self.worker = self.worker, None
        if worker is not None:
            worker.close()
