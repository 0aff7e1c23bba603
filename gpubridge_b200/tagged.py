"""Collectives over a tagged-message worker (``send / recv / wait / abort / close``).

Shared by the host-staged transports whose native worker moves tagged byte ranges (here the
multi-stream TCP worker of ``csrc/gb_tcp.cpp``); same algorithms and guarantees as the
reference's (src/gpubridge/tagged.py:45-230):

* two members: both post every chunk's receive and send at once, then reduce chunk *i* as
  soon as its receive **and** its send have completed (the send reads the same memory),
  while later chunks are still on the wire;
* more members: ring reduce-scatter then ring all-gather over near-equal segments;
* broadcast: the root sends to every other member;
* reductions run on one torch thread; any exception aborts the worker before it propagates,
  so no posted operation outlives the tensors it points into;
* link setup publishes a status key per member on the job's store, so every rank - member or
  not - learns whether the link came up and fails with the same message if not.

Tag layout (64 bits): sequence (24) | step (12) | sender (8) | chunk (20).
"""
from __future__ import annotations

import os
import time
from collections.abc import Sequence
from datetime import timedelta
from typing import Any, ClassVar

import torch

from gpubridge_b200.transport import BridgeTransport, LinkContext

DEFAULT_TIMEOUT = timedelta(minutes=30)
HANDSHAKE_STEP = 0xFFF

#: dtype and op codes of the native collectives (csrc/gb_tcp.cpp)
_NATIVE_DTYPES = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2, torch.float64: 3,
                  torch.int8: 4, torch.uint8: 5, torch.int32: 6, torch.int64: 7}
_NATIVE_OPS = {"sum": 0, "max": 1, "min": 2}


def native_collectives() -> bool:
    """``GPUBRIDGE_TAGGED_NATIVE=0`` keeps the collectives in Python (the oracle of the tests)."""
    return os.environ.get("GPUBRIDGE_TAGGED_NATIVE", "1") != "0"


_REDUCE = {"sum": torch.Tensor.add_, "max": lambda a, b: torch.maximum(a, b, out=a),
           "min": lambda a, b: torch.minimum(a, b, out=a)}


def tag(seq: int, step: int, sender: int, chunk: int) -> int:
    return ((seq & 0xFFFFFF) << 40) | ((step & 0xFFF) << 28) | ((sender & 0xFF) << 20) | \
        (chunk & 0xFFFFF)


def segments(numel: int, parts: int) -> list[tuple[int, int]]:
    """(start, length) of ``parts`` near-equal segments; the first ``numel % parts`` get one more."""
    base, extra = divmod(numel, parts)
    out, start = [], 0
    for i in range(parts):
        length = base + (1 if i < extra else 0)
        out.append((start, length))
        start += length
    return out


def pieces(numel: int, chunk: int) -> list[tuple[int, int]]:
    return [(s, min(chunk, numel - s)) for s in range(0, numel, chunk)] or [(0, 0)]


def wait_for_keys(store, keys: Sequence[str], deadline: float, what: str) -> list[str]:
    while True:
        try:
            store.wait(list(keys), timedelta(seconds=max(0.05, min(2.0, deadline - time.monotonic()))))
            return [store.get(k).decode() for k in keys]
        except Exception:  # noqa: BLE001
            if time.monotonic() >= deadline:
                raise RuntimeError(f"timed out waiting for {what}") from None


class TaggedBridge(BridgeTransport):
    """Subclasses set ``name`` and implement :meth:`_connect`."""

    reduce_ops = frozenset({"sum", "max", "min"})
    _instead: ClassVar[str] = 'use bridge="gloo" to run without it'

    def __init__(self, worker: Any, members: Sequence[int], rank: int, timeout: timedelta,
                 chunk_bytes: int) -> None:
        self.worker = worker
        self.members = list(members)
        self.index = self.members.index(rank)
        self.timeout = timeout.total_seconds()
        self.chunk_bytes = chunk_bytes
        self._seq = 0

    # -- creation ------------------------------------------------------------------------------
    @classmethod
    def create(cls, ranks, *, context: LinkContext, timeout=None):
        timeout = timeout or DEFAULT_TIMEOUT
        members, rank, store = list(ranks), context.rank, context.store
        key = f"gb/{cls.name}/{context.name}/{'_'.join(map(str, members))}"
        deadline = time.monotonic() + timeout.total_seconds()
        transport, error = None, None
        if rank in members:
            try:
                transport = cls._connect(store, key, members, rank, timeout, deadline)
            except Exception as exc:  # noqa: BLE001 - reported to every rank below
                error = f"{type(exc).__name__}: {exc}"
            store.set(f"{key}/status/{rank}", "ok" if error is None else error)
        statuses = wait_for_keys(store, [f"{key}/status/{m}" for m in members], deadline,
                                 f"every bridge member to report on its {cls.name} connections")
        failed = [(m, s) for m, s in zip(members, statuses) if s != "ok"]
        if failed:
            if transport is not None:
                transport.close()
            detail = "\n".join(f"  rank {m}: {s}" for m, s in failed)
            raise RuntimeError(f"The {cls.name} bridge between ranks {members} could not be set "
                               f"up; {cls._instead}.\n{detail}")
        return transport

    @classmethod
    def _connect(cls, store, key, members, rank, timeout, deadline) -> "TaggedBridge":
        raise NotImplementedError

    def _handshake(self, deadline: float) -> None:
        """One small message each way with every other member: a link that cannot carry data
        fails now, not inside the first collective."""
        hello = torch.tensor([self.index], dtype=torch.int64)
        replies, ids = {}, []
        for peer in self._peers():
            replies[peer] = torch.full((1,), -1, dtype=torch.int64)
            ids.append(self.worker.recv(peer, replies[peer].data_ptr(), 8,
                                        tag(0, HANDSHAKE_STEP, peer, 0)))
            ids.append(self.worker.send(peer, hello.data_ptr(), 8,
                                        tag(0, HANDSHAKE_STEP, self.index, 0)))
        self.worker.wait(ids, deadline)
        for peer, reply in replies.items():
            if int(reply) != peer:
                raise RuntimeError(f"{self.name} handshake with bridge member {peer} returned "
                                   f"{int(reply)}")

    # -- plumbing --------------------------------------------------------------------------------
    def _peers(self) -> list[int]:
        return [i for i in range(len(self.members)) if i != self.index]

    def _check(self, tensor: torch.Tensor) -> None:
        if not tensor.is_contiguous() or tensor.device.type != "cpu":
            raise ValueError(f"the {self.name} bridge carries contiguous host tensors")

    def _begin(self, tensor: torch.Tensor) -> tuple[int, float, int]:
        self._seq += 1
        return (self._seq, time.monotonic() + self.timeout,
                max(1, self.chunk_bytes // tensor.element_size()))

    def _post(self, fn, peer: int, view: torch.Tensor, seq: int, step: int, sender: int,
              chunk: int) -> list[int]:
        size = view.element_size()
        return [fn(peer, view.data_ptr() + start * size, length * size, tag(seq, step, sender, i))
                for i, (start, length) in enumerate(pieces(view.numel(), chunk))]

    def _guarded(self, run) -> None:
        threads = torch.get_num_threads()
        torch.set_num_threads(1)
        try:
            run()
        except BaseException:
            self.worker.abort()
            raise
        finally:
            torch.set_num_threads(threads)

    # -- collectives -----------------------------------------------------------------------------
    def all_reduce(self, tensor: torch.Tensor, op: str = "sum") -> None:
        if len(self.members) == 1:
            return
        self._check(tensor)
        self._guarded(lambda: self._all_reduce(tensor, op))

    def _all_reduce(self, tensor: torch.Tensor, op: str) -> None:
        seq, deadline, chunk = self._begin(tensor)
        size, fold = len(self.members), _REDUCE[op]
        flat = tensor.view(-1)
        worker = self.worker
        if (hasattr(worker, "all_reduce") and tensor.dtype in _NATIVE_DTYPES
                and native_collectives()):
            worker.all_reduce(flat.data_ptr(), flat.numel(), _NATIVE_DTYPES[tensor.dtype],
                              _NATIVE_OPS[op], chunk, seq, deadline)
            return
        if size == 2:
            (peer,) = self._peers()
            scratch = torch.empty_like(flat)
            got = self._post(worker.recv, peer, scratch, seq, 0, peer, chunk)
            out = self._post(worker.send, peer, flat, seq, 0, self.index, chunk)
            for (start, length), r, s in zip(pieces(flat.numel(), chunk), got, out):
                worker.wait([r, s], deadline)
                fold(flat[start:start + length], scratch[start:start + length])
            return
        right, left = (self.index + 1) % size, (self.index - 1) % size
        parts = segments(flat.numel(), size)
        scratch = torch.empty(max(length for _, length in parts), dtype=flat.dtype)

        def segment(i: int) -> torch.Tensor:
            start, length = parts[i % size]
            return flat[start:start + length]

        for step in range(size - 1):                       # reduce-scatter
            incoming = segment(self.index - step - 1)
            buffer = scratch[:incoming.numel()]
            ids = self._post(worker.recv, left, buffer, seq, step, left, chunk) + \
                self._post(worker.send, right, segment(self.index - step), seq, step, self.index, chunk)
            worker.wait(ids, deadline)
            fold(incoming, buffer)
        for step in range(size - 1):                       # all-gather: I own segment index + 1
            ids = self._post(worker.recv, left, segment(self.index - step), seq, size + step,
                             left, chunk) + \
                self._post(worker.send, right, segment(self.index + 1 - step), seq, size + step,
                           self.index, chunk)
            worker.wait(ids, deadline)

    def broadcast(self, tensor: torch.Tensor, src: int) -> None:
        if len(self.members) == 1:
            return
        self._check(tensor)
        self._guarded(lambda: self._broadcast(tensor, src))

    def _broadcast(self, tensor: torch.Tensor, src: int) -> None:
        seq, deadline, chunk = self._begin(tensor)
        root = self.members.index(src)
        flat = tensor.view(-1)
        if hasattr(self.worker, "broadcast") and native_collectives():
            self.worker.broadcast(flat.data_ptr(), flat.numel() * flat.element_size(), root,
                                  chunk * flat.element_size(), seq, deadline)
            return
        if self.index == root:
            ids = [i for peer in self._peers()
                   for i in self._post(self.worker.send, peer, flat, seq, 0, root, chunk)]
        else:
            ids = self._post(self.worker.recv, root, flat, seq, 0, root, chunk)
        self.worker.wait(ids, deadline)

    def close(self) -> None:
        worker, self.worker = self.worker, None
        if worker is not None:
            worker.close()
