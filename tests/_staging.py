"""Staging layers that make copy ordering checkable on CPU.

A GPU runs a queued copy whenever its stream gets to it, so a pipeline may rely only on the
events it waits for.  ``DeferredStaging`` takes that literally: a copy is executed only when
somebody waits for its event, or for a later event of the same stream (a stream runs in
order), or when another queued copy names it as its precondition.  A pipeline that forgets a
wait then hands the bridge a slot whose copy never ran, and the result stops matching the
flat-gloo oracle - a wrong answer instead of a race.  (The reference tests its pipeline the
same way: tests/_staging.py there.)
"""
from __future__ import annotations

from collections import deque

import torch

from gpubridge_b200.staging import HostStaging


class Ticket:
    """Stands for a CUDA event: done once the copy it was recorded after has run."""

    def __init__(self, lane: "Lane", label: str) -> None:
        self.lane, self.label, self.done = lane, label, False

    def settle(self) -> None:
        if not self.done:
            self.lane.run_until(self)


class Lane:
    """Stands for a CUDA stream: runs its queued copies in order, only as far as asked."""

    def __init__(self, journal: list) -> None:
        self.journal, self.pending = journal, deque()

    def queue(self, label: str, action, after: Ticket | None) -> Ticket:
        ticket = Ticket(self, label)
        self.pending.append((ticket, action, after))
        return ticket

    def run_until(self, ticket: Ticket) -> None:
        while not ticket.done:
            queued, action, after = self.pending.popleft()
            if after is not None:
                after.settle()          # a stream-side wait: the other lane gets there first
            action()
            queued.done = True
            self.journal.append(("ran", queued.label))


class DeferredStaging(HostStaging):
    """Host slots separate from the tensor, copies deferred, every call journalled."""

    def __init__(self, chunk_bytes: int, slots: int) -> None:
        self.buffers = [torch.full((chunk_bytes,), 0xEE, dtype=torch.uint8) for _ in range(slots)]
        self.journal: list = []
        self.out, self.back = Lane(self.journal), Lane(self.journal)
        self.count = 0

    def slot(self, index, chunk):
        return self.buffers[index][:chunk.numel() * chunk.element_size()].view(chunk.dtype)

    def begin(self, tensor):
        self.journal.append(("begin",))

    def _name(self, kind: str) -> str:
        self.count += 1
        return f"{kind}{self.count}"

    def to_host(self, slot, chunk, after=None):
        label = self._name("out")
        self.journal.append(("to_host", label, after.label if after else None))
        return self.out.queue(label, lambda: slot.copy_(chunk), after)

    def wait_host(self, event):
        self.journal.append(("wait_host", event.label if event else None))
        if event is not None:
            event.settle()

    def to_device(self, chunk, slot):
        label = self._name("back")
        self.journal.append(("to_device", label))
        return self.back.queue(label, lambda: chunk.copy_(slot), None)

    def end(self, event):
        self.journal.append(("end", event.label if event else None))
        if event is not None:
            event.settle()

    def close(self):
        pass


class CallerKeepsGoing(DeferredStaging):
    """``end()`` only makes the caller's stream wait, as on a GPU: the collective returns with
    its copies back still queued; :meth:`caller_reaches_the_waits` is that stream catching up."""

    def __init__(self, chunk_bytes: int, slots: int) -> None:
        super().__init__(chunk_bytes, slots)
        self.owed: list[Ticket] = []

    def end(self, event):
        self.journal.append(("end", event.label if event else None))
        if event is not None:
            self.owed.append(event)

    def caller_reaches_the_waits(self) -> None:
        for ticket in self.owed:
            ticket.settle()
        self.owed.clear()


class SkipsWaitHost(DeferredStaging):
    """A broken staging layer for the negative control: the host never waits for a copy out."""

    def wait_host(self, event):
        self.journal.append(("wait_host-skipped", event.label if event else None))
