"""Host staging for the host-staged (cross-node fallback) bridge.

On one NVSwitch box the bridge is NVLink and nothing here runs.  Across nodes the leaders'
data goes through host memory; these classes order those copies with CUDA events and never
synchronise the whole device (reference: src/gpubridge/staging.py:45-242):

* :class:`ChunkStaging`: pinned slots plus one stream for copies out and one for copies
  back, so chunk k+1 leaves the GPU while chunk k is on the wire and chunk k-1 returns.
* :class:`WholeStaging`: one pinned buffer grown to the largest tensor seen, copies on the
  caller's stream; the copy back is not waited for - its event gates the next copy out.

Both are written against four small device operations (``_allocate``, ``_copy``,
``_wait``, ``_order``) so tests can substitute lazy copies and catch a missing wait as a
wrong answer on CPU.
"""
from __future__ import annotations

import torch

from gpubridge_b200._mutation import mutated


class HostStaging:
    """On CPU a tensor already is host memory: slots are the chunks, copies are no-ops."""

    def slot(self, index: int, chunk: torch.Tensor) -> torch.Tensor:
        return chunk

    def begin(self, tensor: torch.Tensor) -> None:
        pass

    def to_host(self, slot, chunk, after=None):
        return None

    def wait_host(self, event) -> None:
        pass

    def to_device(self, chunk, slot):
        return None

    def end(self, event) -> None:
        pass

    def close(self) -> None:
        pass


class ChunkStaging(HostStaging):
    """``slots`` pinned buffers of ``chunk_bytes`` and two copy streams."""

    def __init__(self, device: torch.device, chunk_bytes: int, slots: int) -> None:
        self.device = device
        self.buffers = [self._allocate(chunk_bytes) for _ in range(slots)]
        self.out_stream = torch.cuda.Stream(device)
        self.back_stream = torch.cuda.Stream(device)

    def _allocate(self, nbytes: int) -> torch.Tensor:
        return torch.empty(nbytes, dtype=torch.uint8, pin_memory=True)

    def slot(self, index, chunk):
        return self.buffers[index][:chunk.numel() * chunk.element_size()].view(chunk.dtype)

    def begin(self, tensor):
        ready = torch.cuda.Event()
        ready.record(torch.cuda.current_stream(self.device))
        for stream in (self.out_stream, self.back_stream):
            if not mutated("staging-ignores-caller"):
                stream.wait_event(ready)
            tensor.record_stream(stream)

    def _copy(self, stream, dst, src, after):
        if after is not None:
            stream.wait_event(after)
        with torch.cuda.stream(stream):
            dst.copy_(src, non_blocking=True)
            done = torch.cuda.Event()
            done.record(stream)
        return done

    def to_host(self, slot, chunk, after=None):
        return self._copy(self.out_stream, slot, chunk, after)

    def wait_host(self, event):
        if event is not None:
            event.synchronize()

    def to_device(self, chunk, slot):
        return self._copy(self.back_stream, chunk, slot, None)

    def end(self, event):
        if event is not None:
            torch.cuda.current_stream(self.device).wait_event(event)

    def close(self):
        self.buffers.clear()


class WholeStaging:
    """One pinned buffer for a leader's whole-tensor bridge step."""

    def __init__(self, device: torch.device) -> None:
        self.device = device
        self.buffer: torch.Tensor | None = None
        self.copied_back = None

    def to_host(self, tensor: torch.Tensor) -> torch.Tensor:
        nbytes = tensor.numel() * tensor.element_size()
        if self.buffer is None or self.buffer.numel() < nbytes:
            if self.copied_back is not None:
                self._wait(self.copied_back)      # the old buffer may still be read
            self.buffer, self.copied_back = self._allocate(nbytes), None
        host = self.buffer[:nbytes].view(tensor.dtype).view(tensor.shape)
        self._wait(self._copy(host, tensor, self.copied_back))   # before the bridge reads it
        return host

    def to_device(self, tensor: torch.Tensor, host: torch.Tensor) -> None:
        self.copied_back = self._copy(tensor, host, None)

    def close(self) -> None:
        if self.copied_back is not None:
            self._wait(self.copied_back)
        self.buffer = self.copied_back = None

    # -- device operations (tests replace these) -------------------------------------------
    def _allocate(self, nbytes: int) -> torch.Tensor:
        return torch.empty(nbytes, dtype=torch.uint8, pin_memory=True)

    def _copy(self, dst, src, after):
        stream = torch.cuda.current_stream(self.device)
        if after is not None:
            stream.wait_event(after)
        dst.copy_(src, non_blocking=True)
        done = torch.cuda.Event()
        done.record(stream)
        return done

    def _wait(self, event) -> None:
        event.synchronize()


def make_bridge_staging(device: torch.device):
    """Whole-tensor pinned staging for ``device``; None on CPU.  Tests replace this."""
    return WholeStaging(device) if device.type == "cuda" else None


def make_staging(device: torch.device, chunk_bytes: int, slots: int):
    """Chunked staging for ``device``.  Tests replace this."""
    if device.type == "cuda":
        return ChunkStaging(device, chunk_bytes, slots)
    return HostStaging()
