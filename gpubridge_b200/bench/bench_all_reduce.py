"""Collective sweep: bus bandwidth of the fused collectives against plain NCCL.

Method (the reference's, scripts/gpu/bench_all_reduce.py:125-197): per size 5 warm-ups, then
up to ``--trials`` timed calls (or ``--seconds``), each bracketed by CUDA events on the
current stream; a trial's latency is the slowest rank's; the median over trials is reported;
``algbw = bytes / t`` and, as nccl-tests does, ``busbw = algbw * 2 (n-1) / n`` for
all_reduce, ``algbw * (n-1) / n`` for all_gather and reduce_scatter, ``algbw`` for broadcast.

Run under torchrun, one process per GPU, e.g.::

    GPUBRIDGE_ISLANDS=4,4 python -m torch.distributed.run --nproc-per-node 8 \
        --master-addr 127.0.0.1 -m gpubridge_b200.bench.bench_all_reduce --largest 1G

Targets: ``ours`` (the active policy), ``nccl`` (one NCCL communicator of every rank),
``policy:<name>`` and ``compression:<mode>[:<format>]`` (a policy instance of their own).
``--write-thresholds PATH`` writes an auto-tuned thresholds file from the measured winners.
"""
from __future__ import annotations

import argparse
import os
import json
import statistics
import sys
import time
import warnings

import torch

import gpubridge_b200 as gb
from gpubridge_b200 import policies as _policies
from gpubridge_b200.config import parse_size
from gpubridge_b200.ops import _lib as _native

BUS = {"all_reduce": lambda n: 2 * (n - 1) / n, "all_gather": lambda n: (n - 1) / n,
       "reduce_scatter": lambda n: (n - 1) / n, "broadcast": lambda n: 1.0}


def sizes(lo: int, hi: int) -> list[int]:
    out, s = [], lo
    while s <= hi:
        out.append(s)
        s *= 2
    return out


def time_calls(fn, topology, trials: int, seconds: float, warmup: int = 5, inner: int = 1,
               graph: bool = False) -> float:
    """Median over trials of the slowest rank's device time per call, in milliseconds.  With
    ``inner`` > 1 a trial is that many back-to-back calls (what a training step issues), which
    takes the launch and host jitter of a lone call out of small-message latencies.  With
    ``graph`` the ``inner`` calls are captured once in a CUDA graph and a trial is one replay:
    what the device needs, with no host work between the calls."""
    dev = topology.device
    on_gpu = dev.type == "cuda"
    for _ in range(warmup):
        fn()
    if on_gpu:
        torch.cuda.synchronize(dev)
    topology.world_group.barrier()
    if graph and on_gpu:
        captured = torch.cuda.CUDAGraph()
        here = torch.cuda.current_stream(dev)
        side = here if here != torch.cuda.default_stream(dev) else torch.cuda.Stream(dev)
        with torch.cuda.graph(captured, stream=side):       # never the default stream
            for _ in range(inner):
                fn()
        torch.cuda.synchronize(dev)
        topology.world_group.barrier()
        run_trial = captured.replay
    else:
        def run_trial():
            for _ in range(inner):
                fn()
    times, started = [], time.monotonic()
    for _ in range(trials):
        if on_gpu:
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            run_trial()
            end.record()
            end.synchronize()
            took = start.elapsed_time(end)
        else:                                   # CPU simulation: the host clock
            t0 = time.perf_counter()
            for _ in range(inner):
                fn()
            took = (time.perf_counter() - t0) * 1e3
        slowest = torch.tensor([took / inner], dtype=torch.float64)
        topology.world_group.all_reduce(slowest, "max")
        times.append(float(slowest))
        stop = torch.tensor([1.0 if time.monotonic() - started > seconds else 0.0])
        topology.world_group.all_reduce(stop, "max")
        if float(stop) > 0:
            break
    return statistics.median(times)


_made: dict[str, object] = {}           # target name -> its policy, set up once per job


def target_policy(name: str, topology):
    """The policy behind a target: the job's own, or one set up for ``policy:NAME`` /
    ``compression:MODE[:FORMAT]`` - once, whatever the number of sizes (setting a policy up is
    collective and may build communicators)."""
    if not (name.startswith("policy:") or name.startswith("compression:")):
        return topology.policy
    if name not in _made:
        if name.startswith("policy:"):
            cls = _policies.choose_policy(_policies.resolve_policy(name.split(":", 1)[1]), topology.layout)
            policy = cls()
            policy.setup(topology)
        else:
            parts = name.split(":")
            policy = type(topology.policy)(compression=parts[1]) if hasattr(
                topology.policy, "compression") else topology.policy
            policy.setup(topology)
            if len(parts) > 2:
                policy._fmt = parts[2]
        _made[name] = policy
    return _made[name]


def close_targets(topology) -> None:
    for policy in _made.values():
        if policy is not topology.policy:
            policy.close()
    _made.clear()


_heap = None
_heap_bytes = 0


def make_target(name: str, op: str, topology, dtype, nbytes: int):
    """A zero-argument callable running ``op`` once on ``nbytes`` of ``dtype``."""
    dev, world = topology.device, topology.world_size
    n = max(1, nbytes // torch.empty(0, dtype=dtype).element_size())
    gen = torch.Generator(device="cpu").manual_seed(1234 + topology.rank)
    full = torch.randn(n, generator=gen).to(dtype).to(dev)
    if name == "nccl":
        comm = topology.p2p_group
        if op == "all_reduce":
            return lambda: comm.all_reduce(full), nbytes
        if op == "broadcast":
            return lambda: comm.broadcast(full, topology.layout.members[0]), nbytes
        part = full[: n // world]
        if op == "all_gather":
            out = torch.empty(part.numel() * world, dtype=dtype, device=dev)
            return lambda: comm.all_gather_into(out, part), out.nbytes
        out = torch.empty(n // world, dtype=dtype, device=dev)
        src = full[: out.numel() * world]
        return lambda: comm.reduce_scatter_into(out, src), src.nbytes
    if name == "ours-native":
        # the native engine's own entry point, as the C++ front end calls it (planner and launch
        # in C++, no Python policy layer): what DDP's hook and FSDP2 get per call
        fabric = topology.fabric
        engine = fabric.engine() if fabric is not None and op == "all_reduce" else 0
        if not engine or dtype not in _native.DTYPES:
            return None, nbytes
        lib, code = fabric.lib, _native.DTYPES[dtype]
        ptr, count = full.data_ptr(), full.numel()

        def native_call(keep=full):            # the closure owns the tensor: only its address is used
            stream = torch.cuda.current_stream(dev).cuda_stream
            _native.check(lib.gb_engine_all_reduce(engine, ptr, ptr, count, code, 0, 0, 0, stream),
                          "gb_engine_all_reduce")
        return native_call, nbytes
    if name == "ours-inplace":
        # the tensor lives in the team's switch memory (what the data-parallel trainer does
        # with its gradients): the all-reduce runs in place inside the NVSwitch, nothing staged
        fabric = topology.fabric
        if op != "all_reduce" or fabric is None or not hasattr(fabric, "switch_empty"):
            return None, nbytes
        global _heap
        if _heap is None or _heap.numel() * _heap.element_size() < nbytes:
            _heap = fabric.switch_empty(max(nbytes, _heap_bytes) // 4, torch.float32)
        if _heap is None:
            return None, nbytes
        home = _heap.view(torch.uint8)[:nbytes].view(dtype)
        home.copy_(full)
        policy = topology.policy
        return lambda: policy.all_reduce(home, topology), nbytes
    policy = target_policy(name, topology)
    if op == "all_reduce":
        return lambda: policy.all_reduce(full, topology), nbytes
    if op == "broadcast":
        return lambda: policy.broadcast(full, topology.layout.members[0], topology), nbytes
    part = full[: n // world]
    if op == "all_gather":
        out = torch.empty(part.numel() * world, dtype=dtype, device=dev)
        return lambda: policy.all_gather_into_tensor(out, part, topology), out.nbytes
    out = torch.empty(n // world, dtype=dtype, device=dev)
    src = full[: out.numel() * world]
    return lambda: policy.reduce_scatter_tensor(out, src, topology), src.nbytes


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--smallest", default="4K", help="smallest payload")
    ap.add_argument("--largest", default="64M", help="largest payload")
    ap.add_argument("--ops", default="all_reduce")
    ap.add_argument("--targets", default="ours,nccl")
    ap.add_argument("--dtypes", default="float32")
    ap.add_argument("--trials", type=int, default=20)
    ap.add_argument("--seconds", type=float, default=20.0)
    ap.add_argument("--inner", type=int, default=1, help="back-to-back calls per trial")
    ap.add_argument("--json", default="")
    ap.add_argument("--graph", action="store_true", help="capture the --inner calls of a trial in "
                    "a CUDA graph and time its replay (device time without host work between calls)")
    ap.add_argument("--blocks", type=int, default=0, help="cap the grid of this library's kernels "
                    "(what a collective that runs beside compute gets)")
    ap.add_argument("--bridge", default=os.environ.get("GPUBRIDGE_BRIDGE", "").strip() or None,
                    help="bridge transport between islands (default: GPUBRIDGE_BRIDGE, else init()'s choice)")
    ap.add_argument("--write-thresholds", default="")
    ap.add_argument("--candidates", default="", help="policies to race at every size (adds a "
                    "policy:NAME target for each; with --write-thresholds the winners become the rules)")
    ap.add_argument("--phases", action="store_true", help="for the target `ours`: the phases of the "
                    "all-reduce through the public API with an observer attached - the slowest rank's "
                    "median per phase (device timestamps inside the fused kernel, stream events around "
                    "the steps of the composed path)")
    args = ap.parse_args(argv)
    if args.candidates:
        args.targets = ",".join([*filter(None, args.targets.split(",")),
                                 *(f"policy:{name}" for name in args.candidates.split(","))])

    with warnings.catch_warnings():
        warnings.simplefilter("ignore", gb.SplitTestWarning)
        topology = gb.init(**({"bridge": args.bridge} if args.bridge else {}))
    rank, world = topology.rank, topology.world_size
    rows = []
    global _heap_bytes
    _heap_bytes = parse_size(args.largest)
    import contextlib
    capped = (lambda: topology.fabric.grid_cap(args.blocks)) if args.blocks and topology.fabric is not None \
        else contextlib.nullcontext
    try:
        for op in args.ops.split(","):
            for dtype_name in args.dtypes.split(","):
                dtype = getattr(torch, dtype_name)
                for nbytes in sizes(parse_size(args.smallest), parse_size(args.largest)):
                    for target in args.targets.split(","):
                        if target == "nccl" and topology.p2p_group is None:
                            continue
                        fn, moved = make_target(target, op, topology, dtype, nbytes)
                        if fn is None:
                            continue
                        # the fused kernels are timed on the stream they run on, as the async
                        # (DDP / FSDP) path uses them; NCCL is timed on the current stream
                        fused = target != "nccl" and topology.fabric is not None
                        if topology.device.type == "cuda":
                            stream = (topology.fabric.comm_stream if fused
                                      else torch.cuda.current_stream(topology.device))
                            with torch.cuda.stream(stream), (capped() if fused else contextlib.nullcontext()):
                                ms = time_calls(fn, topology, args.trials, args.seconds,
                                                inner=args.inner, graph=args.graph)
                        else:
                            ms = time_calls(fn, topology, args.trials, args.seconds, inner=args.inner)
                        algbw = moved / (ms * 1e-3) / 1e9
                        row = {"op": op, "dtype": dtype_name, "bytes": moved, "target": target,
                               "ms": round(ms, 5), "algbw_gbs": round(algbw, 3),
                               "busbw_gbs": round(algbw * BUS[op](world), 3), "world": world,
                               "islands": [len(i.ranks) for i in topology.layout.islands],
                               "policy": topology.policy_name, "inner": args.inner}
                        if args.blocks and fused:
                            row["blocks"] = args.blocks
                        if args.graph:
                            row["graph"] = True
                        if target.startswith("compression:") and op == "all_reduce":
                            row.update(compression_check(target, topology, dtype, nbytes))
                        if args.phases and target == "ours" and op == "all_reduce":
                            row["phases_ms"] = phase_times(topology, dtype, nbytes, min(args.trials, 10))
                        rows.append(row)
                        if rank == 0:
                            print(json.dumps(row), flush=True)
        if topology.fabric is not None:
            topology.fabric.check()
    finally:
        close_targets(topology)
        gb.destroy()
    if rank == 0 and args.json:
        with open(args.json, "w") as fh:
            json.dump(rows, fh, indent=1)
    if rank == 0 and args.write_thresholds:
        write_thresholds(rows, args.write_thresholds)
    return 0


class _Records(gb.CollectiveObserver):
    def __init__(self) -> None:
        self.records = []

    def on_collective(self, record) -> None:
        self.records.append(record)


def phase_times(topology, dtype, nbytes: int, trials: int) -> dict[str, float]:
    """``{phase: ms}``: all-reduces through the public API with an observer attached; per
    phase the median over the trials, then the slowest rank's (ranks that do not take part in
    a phase - members during the bridge step - do not report it)."""
    import torch.distributed as dist
    dev = topology.device
    n = max(1, nbytes // torch.empty(0, dtype=dtype).element_size())
    t = torch.ones(n, dtype=dtype, device=dev)
    watcher = _Records()
    gb.all_reduce(t)                                          # warm
    gb.add_observer(watcher)
    try:
        for _ in range(trials):
            gb.all_reduce(t)
        if dev.type == "cuda":
            torch.cuda.synchronize(dev)
    finally:
        gb.remove_observer(watcher)
    seen: dict[str, list[float]] = {}
    for record in watcher.records:
        seen.setdefault("total", []).append(gb.elapsed_ms(record.start, record.end))
        for phase in record.phases:
            seen.setdefault(phase.name, []).append(phase.elapsed_ms())
    mine = {name: statistics.median(values) for name, values in seen.items()}
    everyone = [None] * topology.world_size
    dist.all_gather_object(everyone, mine)
    names = sorted({name for m in everyone for name in m})
    return {name: round(max(m[name] for m in everyone if name in m), 5) for name in names}


def compression_check(target: str, topology, dtype, nbytes: int) -> dict:
    """One compressed all-reduce of fresh data against the fp64 sum: the largest error relative
    to the largest magnitude of the result, and whether every rank holds identical bits (the
    reference's ``--compression`` check, scripts/gpu/bench_all_reduce.py:331-379)."""
    dev, world = topology.device, topology.world_size
    n = max(1, nbytes // torch.empty(0, dtype=dtype).element_size())
    inputs = [torch.randn(n, generator=torch.Generator().manual_seed(99 + r)).to(dtype)
              for r in range(world)]
    exact = torch.stack([t.double() for t in inputs]).sum(0)
    mine = inputs[topology.rank].to(dev)
    policy = target_policy(target, topology)
    policy.all_reduce(mine, topology)
    if dev.type == "cuda":
        torch.cuda.synchronize(dev)
    got = mine.cpu()
    error = float((got.double() - exact).abs().max() / exact.abs().max().clamp_min(1e-30))
    bits = got.view(torch.uint8).to(torch.int32)
    hi, lo = bits.clone(), bits.clone()
    topology.world_group.all_reduce(hi, "max")
    topology.world_group.all_reduce(lo, "min")
    return {"max_rel_error": round(error, 6), "identical_bits": bool(torch.equal(hi, lo))}


def write_thresholds(rows: list[dict], path: str) -> None:
    """The fastest ``policy:*`` target per size becomes a rule; neighbouring sizes with the
    same winner are merged; the last rule covers every size."""
    best: dict[int, tuple[float, str]] = {}
    for row in rows:
        if row["op"] != "all_reduce" or not row["target"].startswith("policy:"):
            continue
        name = row["target"].split(":", 1)[1]
        if row["bytes"] not in best or row["ms"] < best[row["bytes"]][0]:
            best[row["bytes"]] = (row["ms"], name)
    rules: list[dict] = []
    for size in sorted(best):
        name = best[size][1]
        if rules and rules[-1]["policy"] == name:
            rules[-1]["max_bytes"] = size
        else:
            rules.append({"max_bytes": size, "policy": name})
    if not rules:
        rules = [{"max_bytes": None, "policy": "auto"}]
    rules[-1]["max_bytes"] = None
    _policies.write_thresholds(path, rules, _policies.PipelinedReduceBridgeBroadcast
                               .DEFAULT_CHUNK_BYTES)


if __name__ == "__main__":
    sys.exit(main())
