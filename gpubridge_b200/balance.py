"""Pipeline stage balancing (opt-in; nothing else imports it).

Same contract as the reference's ``gpubridge.balance`` (src/gpubridge/balance.py:36-268):
profile each layer on a stage's device (forward, backward, output bytes, state bytes, saved
activation bytes, one microbatch), then cut the layers into contiguous stages so that the
slowest stage - its own layers plus ``2 * bytes / bandwidth`` at every boundary it shares
with a neighbour - is as fast as possible, within each stage's memory (state plus saved
activations times the microbatches in flight: all of them under GPipe, ``stages - stage``
under 1F1B).  The search is exact and deterministic, so every rank computes the same split.

The search here runs from the last stage backwards with memoisation
(``tail(s, i)`` = best bottleneck of stages ``s..`` holding layers ``i..``), which visits the
same ``O(stages * layers^2)`` states as a forward table.
"""
from __future__ import annotations

import copy
import functools
import statistics
import time
from collections.abc import Sequence
from dataclasses import dataclass

import torch
from torch import nn

__all__ = ["LayerCost", "Plan", "evaluate", "in_flight", "partition", "profile_layers"]


@dataclass(frozen=True)
class LayerCost:
    """One layer on one device, one microbatch."""

    forward_ms: float
    backward_ms: float
    out_bytes: int
    state_bytes: int
    activation_bytes: int

    @property
    def ms(self) -> float:
        return self.forward_ms + self.backward_ms


@dataclass(frozen=True)
class Plan:
    split: list[int]
    stage_ms: list[float]
    bottleneck_ms: float


def in_flight(schedule: str, stages: int, microbatches: int) -> list[int]:
    """Microbatches whose activations each stage holds at once."""
    if stages < 1 or microbatches < 1:
        raise ValueError(f"a schedule needs at least one stage and one microbatch, got {stages} and {microbatches}")
    if schedule == "gpipe":
        return [microbatches] * stages
    if schedule == "1f1b":
        return [min(stages - s, microbatches) for s in range(stages)]
    raise ValueError(f"unknown schedule {schedule!r}")


def _clock(device: torch.device):
    """``run(fn) -> (result, milliseconds)`` on the device's own clock."""
    if device.type != "cuda":
        def run(fn):
            t0 = time.perf_counter()
            out = fn()
            return out, (time.perf_counter() - t0) * 1e3
        return run

    def run(fn):
        with torch.cuda.device(device):
            stream = torch.cuda.current_stream()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream)
            out = fn()
            b.record(stream)
            b.synchronize()
        return out, a.elapsed_time(b)
    return run


def _storages(t: torch.Tensor) -> list[tuple[int, int]]:
    """(address, bytes) of every storage a saved tensor keeps alive."""
    if t.layout == torch.sparse_coo:
        parts = [t._indices(), t._values()]
    elif t.layout in (torch.sparse_csr, torch.sparse_bsr):
        parts = [t.crow_indices(), t.col_indices(), t.values()]
    elif t.layout in (torch.sparse_csc, torch.sparse_bsc):
        parts = [t.ccol_indices(), t.row_indices(), t.values()]
    else:
        parts = [t]
    return [(p.untyped_storage().data_ptr(), p.untyped_storage().nbytes()) for p in parts]


def profile_layers(layers: Sequence[nn.Module], example: torch.Tensor, device: torch.device, *,
                   trials: int = 3, warmup: int = 1,
                   state_bytes_per_parameter: int = 16) -> list[LayerCost]:
    """Profile every layer as a *copy* on ``device``, one after another; the layers themselves
    are never moved or run, and the random number generators are restored.  ``example`` feeds
    the first layer, each output feeds the next.  16 bytes per parameter is fp32 weights,
    gradients and AdamW's two moments.  Saved activations count each storage once and leave
    out the layer's own parameters."""
    run = _clock(device)
    costs: list[LayerCost] = []
    with torch.random.fork_rng(devices=[device] if device.type == "cuda" else []):
        x = example.to(device)
        for layer in layers:
            clone = copy.deepcopy(layer)
            for p in clone.parameters():
                p.grad = None
            clone.to(device)
            mine = {p.untyped_storage().data_ptr() for p in clone.parameters()}
            fwd, bwd, kept_bytes = [], [], []
            out = None
            for trial in range(warmup + trials):
                inp = x.detach().requires_grad_(x.is_floating_point())
                kept: dict[int, int] = {}

                def pack(t, kept=kept):
                    for address, size in _storages(t):
                        if address not in mine:
                            kept[address] = size
                    return t

                with torch.autograd.graph.saved_tensors_hooks(pack, lambda t: t):
                    out, f_ms = run(lambda: clone(inp))
                seed = torch.ones_like(out)
                _, b_ms = run(lambda: out.backward(seed))
                if trial >= warmup:
                    fwd.append(f_ms)
                    bwd.append(b_ms)
                    kept_bytes.append(sum(kept.values()))
            n_params = sum(p.numel() for p in clone.parameters())
            costs.append(LayerCost(round(statistics.median(fwd), 4),
                                   round(statistics.median(bwd), 4),
                                   out.numel() * out.element_size(),
                                   n_params * state_bytes_per_parameter, max(kept_bytes)))
            x = out.detach()
            del clone
    return costs


def _shape(layer_ms, boundary_bytes, bytes_per_ms) -> tuple[int, int]:
    stages = len(layer_ms)
    layers = len(layer_ms[0]) if stages else 0
    if stages < 1 or layers < stages or any(len(row) != layers for row in layer_ms):
        raise ValueError(f"need a time for each of at least {stages} layers on each of "
                         f"{stages} stages")
    if len(boundary_bytes) != layers - 1 or len(bytes_per_ms) != stages - 1:
        raise ValueError("need one boundary size per pair of neighbouring layers and one "
                         "bandwidth per pair of neighbouring stages")
    return stages, layers


def _stage_time(s, lo, hi, stages, sums, boundary_bytes, bytes_per_ms) -> float:
    t = sums[s][hi] - sums[s][lo]
    if s > 0:
        t += 2 * boundary_bytes[lo - 1] / bytes_per_ms[s - 1]
    if s < stages - 1:
        t += 2 * boundary_bytes[hi - 1] / bytes_per_ms[s]
    return t


def _prefix(values) -> list[float]:
    out = [0.0]
    for v in values:
        out.append(out[-1] + v)
    return out


def evaluate(split: Sequence[int], layer_ms: Sequence[Sequence[float]],
             boundary_bytes: Sequence[float], bytes_per_ms: Sequence[float]) -> list[float]:
    """Each stage's time per microbatch for a given split.  ``layer_ms[s][i]``: layer ``i`` on
    stage ``s``'s device; ``boundary_bytes[i]``: what crosses between layers ``i`` and ``i+1``;
    ``bytes_per_ms[s]``: the link between stages ``s`` and ``s+1``."""
    stages, layers = _shape(layer_ms, boundary_bytes, bytes_per_ms)
    if len(split) != stages or sum(split) != layers or min(split) < 1:
        raise ValueError(f"split {list(split)}: need {stages} positive counts adding up to "
                         f"{layers}")
    sums = [_prefix(row) for row in layer_ms]
    times, lo = [], 0
    for s, count in enumerate(split):
        times.append(_stage_time(s, lo, lo + count, stages, sums, boundary_bytes, bytes_per_ms))
        lo += count
    return times


def partition(layer_ms: Sequence[Sequence[float]], boundary_bytes: Sequence[float],
              bytes_per_ms: Sequence[float], *, state_bytes: Sequence[int] | None = None,
              activation_bytes: Sequence[int] | None = None,
              in_flight: Sequence[int] | None = None,
              memory_bytes: Sequence[float | None] | None = None) -> Plan:
    """The contiguous split whose slowest stage is fastest, each stage within
    ``memory_bytes[s]`` if given (None: no limit).  Raises ``ValueError`` if nothing fits."""
    stages, layers = _shape(layer_ms, boundary_bytes, bytes_per_ms)
    limited = memory_bytes is not None
    if limited and not (state_bytes and activation_bytes and in_flight):
        raise ValueError("a memory limit needs state_bytes, activation_bytes and in_flight")
    sums = [_prefix(row) for row in layer_ms]
    state = _prefix(state_bytes) if limited else []
    saved = _prefix(activation_bytes) if limited else []
    inf = float("inf")

    def fits(s: int, lo: int, hi: int) -> bool:
        if not limited or memory_bytes[s] is None:
            return True
        need = state[hi] - state[lo] + in_flight[s] * (saved[hi] - saved[lo])
        return need <= memory_bytes[s]

    @functools.lru_cache(maxsize=None)
    def tail(s: int, lo: int) -> tuple[float, int]:
        """(bottleneck, layers of stage s) for stages s.. holding layers lo.."""
        if s == stages - 1:
            if not fits(s, lo, layers):
                return inf, layers - lo
            return _stage_time(s, lo, layers, stages, sums, boundary_bytes, bytes_per_ms), layers - lo
        best, best_count = inf, 1
        # leave at least one layer for every later stage; smaller counts win ties, which
        # matches filling earlier stages first when scanned from the front
        for hi in range(lo + 1, layers - (stages - 1 - s) + 1):
            if not fits(s, lo, hi):
                continue
            rest = tail(s + 1, hi)[0]
            if rest == inf:
                continue
            value = max(_stage_time(s, lo, hi, stages, sums, boundary_bytes, bytes_per_ms), rest)
            if value < best:
                best, best_count = value, hi - lo
        return best, best_count

    if tail(0, 0)[0] == inf:
        raise ValueError("no split fits every stage's memory")
    split, lo = [], 0
    for s in range(stages):
        count = tail(s, lo)[1]
        split.append(count)
        lo += count
    times = evaluate(split, layer_ms, boundary_bytes, bytes_per_ms)
    return Plan(split, times, max(times))
