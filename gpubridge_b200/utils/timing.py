"""Timing a multi-rank region the way every number in this repository is taken: warm-up done by
the caller, a barrier and a device synchronise on both sides, CUDA events on the launching
stream, and the slowest rank counts."""
from __future__ import annotations

import time
from typing import Callable

import torch


def device_time(run: Callable[[int], None], steps: int, device: torch.device,
                barrier: Callable[[], None] | None = None) -> float:
    """Milliseconds ``run(steps)`` takes on ``device`` (host clock on CPU)."""
    on_gpu = device.type == "cuda"
    if on_gpu:
        torch.cuda.synchronize(device)
    if barrier is not None:
        barrier()
    if on_gpu:
        torch.cuda.synchronize(device)
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        run(steps)
        end.record()
        torch.cuda.synchronize(device)
        took = start.elapsed_time(end)
    else:
        t0 = time.perf_counter()
        run(steps)
        took = (time.perf_counter() - t0) * 1e3
    if barrier is not None:
        barrier()
    return took


def max_over_ranks(value: float, topology=None) -> float:
    """The largest ``value`` over the ranks of ``topology`` (the initialised one by default)."""
    if topology is None:
        from gpubridge_b200.topology import get_topology, is_initialized
        if not is_initialized():
            return value
        topology = get_topology()
    if topology.world_size == 1:
        return value
    t = torch.tensor([value], dtype=torch.float64)
    topology.world_group.all_reduce(t, "max")
    return float(t)


def human_bytes(n: int) -> str:
    for unit, size in (("G", 1 << 30), ("M", 1 << 20), ("K", 1 << 10)):
        if n >= size and n % size == 0:
            return f"{n // size}{unit}"
    return str(n)
