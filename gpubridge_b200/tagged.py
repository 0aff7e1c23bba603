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


def wait_for_keys(store, keys: Sequence[str], deadline: float, what: str) -> list[str]:
    """Values of ``keys`` once all exist; polls in short slices so the deadline is honoured
    whatever timeout type the store raises."""
    wanted = list(keys)
    while True:
        slice_s = max(0.05, min(2.0, deadline - time.monotonic()))
        try:
            store.wait(wanted, timedelta(seconds=slice_s))
        except Exception:  # noqa: BLE001
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
