"""Per-call host cost of small all-reduces, in CPU simulation.

    python -m gpubridge_b200.bench.bench_per_call [--out per_call.json]
    python -m gpubridge_b200.bench.bench_per_call --stub-comm          # this package's own work only
    python -m gpubridge_b200.bench.bench_per_call --vendors nvidia,nvidia --policies native-only

One CPU process per rank (Gloo everywhere, ``GPUBRIDGE_VENDOR`` per rank): the numbers are
what the Python layers add to a call, not what a GPU collective costs.  Per policy, for sync
and async calls, without an observer and with one that does nothing, every rank times
``all_reduce`` of one float on its own clock; the cases are interleaved over ``--rounds`` so
drift spreads evenly; rank 0's medians are reported next to one plain all-reduce on the
world's host communicator.  ``--stub-comm`` makes every communicator call return at once
after start-up, leaving checks, policy dispatch, phases and (async) the worker thread.
``--profile N`` adds, for rank 0, the N functions with the most own time over one more round of
synchronous calls (cProfile; the profiler itself makes every call slower, so read shares, not
absolutes).  Counterpart of the reference's ``scripts/bench_per_call.py``.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import tempfile
import time
from pathlib import Path

import torch
import torch.multiprocessing as mp

SETTINGS = ("GPUBRIDGE_BRIDGE_COMPRESSION", "GPUBRIDGE_PINNED_STAGING", "GPUBRIDGE_CHUNK_BYTES",
            "GPUBRIDGE_THRESHOLDS", "GPUBRIDGE_SPLIT_TEST", "GPUBRIDGE_ISLANDS")


def _stub() -> None:
    from gpubridge_b200 import groups
    for name in ("all_reduce", "reduce", "broadcast", "all_gather_into", "reduce_scatter_into",
                 "gather", "scatter", "barrier"):
        setattr(groups.Comm, name, lambda self, *a, **k: None)


def _hot_functions(fn, calls: int, top: int) -> list[dict]:
    import cProfile
    import pstats
    profiler = cProfile.Profile()
    profiler.enable()
    for _ in range(calls):
        fn()
    profiler.disable()
    stats = pstats.Stats(profiler)
    rows = sorted(stats.stats.items(), key=lambda kv: -kv[1][2])[:top]          # by own time
    return [{"function": f"{os.path.basename(file)}:{line}({name})", "calls_per_call": round(nc / calls, 2),
             "own_us_per_call": round(tt / calls * 1e6, 2), "cumulative_us_per_call": round(ct / calls * 1e6, 2)}
            for (file, line, name), (cc, nc, tt, ct, _) in rows]


def _rank(rank: int, vendors, policies, calls, rounds, stub, rendezvous, out, profile=0) -> None:
    os.environ["GPUBRIDGE_VENDOR"] = vendors[rank]
    import gpubridge_b200 as gb

    class Quiet(gb.CollectiveObserver):
        def on_collective(self, record) -> None:
            pass

    results: dict[str, list[float]] = {}
    for policy in policies:
        topo = gb.init(init_method=f"file://{rendezvous}-{policy}", rank=rank,
                       world_size=len(vendors), policy=policy)
        t = torch.ones(1)
        if stub:
            _stub()
        cases = [(mode, watched) for mode in ("sync", "async") for watched in (False, True)]
        quiet = Quiet()
        for _ in range(rounds):
            for mode, watched in cases:
                if watched:
                    gb.add_observer(quiet)
                start = time.perf_counter()
                for _ in range(calls):
                    if mode == "sync":
                        gb.all_reduce(t)
                    else:
                        gb.all_reduce(t, async_op=True).wait()
                per_call = (time.perf_counter() - start) / calls
                if watched:
                    gb.remove_observer(quiet)
                results.setdefault(f"{policy}/{mode}/{'observer' if watched else 'plain'}", []).append(per_call)
            if not stub and topo.cpu_group is not None:
                start = time.perf_counter()
                for _ in range(calls):
                    topo.cpu_group.all_reduce(t, "sum")
                results.setdefault(f"{policy}/bare-world-call", []).append(
                    (time.perf_counter() - start) / calls)
        if profile:
            # every rank makes the calls (they are collectives); rank 0 keeps the profile
            hot = _hot_functions(lambda: gb.all_reduce(t), calls, profile)
            if rank == 0:
                results[f"{policy}/profile"] = hot
        gb.destroy()
        if stub:
            import importlib
            from gpubridge_b200 import groups
            importlib.reload(groups)
    if rank == 0:
        Path(out).write_text(json.dumps({k: v if k.endswith("/profile") else statistics.median(v) * 1e6
                                         for k, v in results.items()}))


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--vendors", default="nvidia,nvidia,amd,amd")
    ap.add_argument("--policies", default="reduce-bridge-broadcast,flat-gloo,pipelined-reduce-bridge-broadcast,sharded-bridge")
    ap.add_argument("--calls", type=int, default=200)
    ap.add_argument("--rounds", type=int, default=5)
    ap.add_argument("--stub-comm", action="store_true")
    ap.add_argument("--profile", type=int, default=0, metavar="N",
                    help="rank 0: the N functions with the most own time per synchronous call")
    ap.add_argument("--out", type=Path)
    args = ap.parse_args(argv)
    set_now = [name for name in SETTINGS if os.environ.get(name)]
    if set_now:
        raise SystemExit(f"unset {', '.join(set_now)}: they change what a policy does per call")
    vendors = args.vendors.split(",")
    policies = [p for p in args.policies.split(",") if p]
    if len(set(vendors)) == 1:          # one island: only the policies that apply to it
        policies = [p for p in policies if p in ("native-only", "flat-gloo")] or ["native-only"]
    else:
        policies = [p for p in policies if p != "native-only"]
    with tempfile.TemporaryDirectory() as tmp:
        result = os.path.join(tmp, "result.json")
        mp.spawn(_rank, args=(vendors, policies, args.calls, args.rounds, args.stub_comm,
                              os.path.join(tmp, "rdv"), result, args.profile), nprocs=len(vendors))
        medians = json.loads(Path(result).read_text())
    profiles = {k: medians.pop(k) for k in [k for k in medians if k.endswith("/profile")]}
    record = {"vendors": vendors, "calls": args.calls, "rounds": args.rounds,
              "stub_comm": args.stub_comm, "torch": torch.__version__,
              "cpus": os.cpu_count(), "us_per_call": medians, "profiles": profiles}
    print(f"{'case':<48} us per call")
    for key, value in medians.items():
        print(f"{key:<48} {value:9.1f}")
    for key, rows in profiles.items():
        print(f"\n{key}: own time per call")
        for row in rows:
            print(f"  {row['own_us_per_call']:8.2f} us  x{row['calls_per_call']:<5} {row['function']}")
    if args.out:
        args.out.parent.mkdir(parents=True, exist_ok=True)
        args.out.write_text(json.dumps(record, indent=1))
    return 0


if __name__ == "__main__":
    sys.exit(main())
