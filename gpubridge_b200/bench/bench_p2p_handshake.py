"""What the host-staged point-to-point engine costs beyond the bytes: store traffic, CPU time
and threads of the handshake, the loop and the health probe.  CPU only.

    python -m gpubridge_b200.bench.bench_p2p_handshake [--store tcp|file] [--iterations 2000]

Two processes, each an :class:`gpubridge_b200.p2p.Engine` on its own client of one c10d store
(wrapped in the ``PrefixStore`` the backend gives its engine).  The link between them
completes every transfer at once and moves nothing, so what is left is the engine's own
work.  Phases, per rank: store calls by method, user + system CPU seconds, wall time, threads.

* ``pingpong``: rank 0 sends, rank 1 sends back, ``--iterations`` times; the one-way time is
  half of rank 0's median round trip - the handshake's latency floor;
* ``idle``: both engines idle for ``--idle`` seconds: an idle engine should cost nothing
  (no store probes, no wake-ups);
* ``missing``: rank 0 starts ``--missing`` sends to a rank that never posts and, while they
  wait, times one ready exchange with rank 1 (waiting lanes must not slow a live one), holds
  for ``--hold`` seconds (what waiting costs per second), then closes (bounded).

Counterpart of the reference's scripts/bench_p2p_handshake.py, for this repository's engine.
One machine, CPU processes: not evidence about GPUs or networks.
"""
from __future__ import annotations

import argparse
import collections
import json
import os
import resource
import statistics
import sys
import tempfile
import threading
import time
from datetime import timedelta

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


class CountingStore:
    """Counts the calls the engine makes on its store."""

    def __init__(self, store) -> None:
        self.store, self.calls = store, collections.Counter()

    def __getattr__(self, name):
        target = getattr(self.store, name)

        def counted(*args, **kwargs):
            self.calls[name] += 1
            return target(*args, **kwargs)
        return counted


class Done:
    def wait(self, timeout=None):
        return True

    def is_completed(self):
        return True


class InstantLink:
    """Every post is complete at once; nothing is moved."""

    def post(self, buffer, peer, tag, sending):
        return Done()

    def close(self):
        pass


def usage() -> float:
    r = resource.getrusage(resource.RUSAGE_SELF)
    return r.ru_utime + r.ru_stime


class Phase:
    def __init__(self, store: CountingStore) -> None:
        self.store = store

    def __enter__(self):
        self.calls, self.cpu, self.wall = collections.Counter(self.store.calls), usage(), time.perf_counter()
        return self

    def __exit__(self, *exc):
        now = collections.Counter(self.store.calls)
        now.subtract(self.calls)
        self.result = {"store_calls": {k: v for k, v in now.items() if v}, "cpu_s": round(usage() - self.cpu, 4),
                       "wall_s": round(time.perf_counter() - self.wall, 4), "threads": threading.active_count()}


def worker(rank: int, args, path: str, out) -> None:
    from gpubridge_b200 import p2p
    torch.set_num_threads(1)
    if args.store == "tcp":
        base = dist.TCPStore("127.0.0.1", args.port, 2, rank == 0, timedelta(seconds=60), wait_for_workers=False)
    else:
        base = dist.FileStore(path, 2)
    store = CountingStore(dist.PrefixStore("p2p-bench", base))
    engine = p2p.Engine(InstantLink(), torch.device("cpu"), rank, store, timedelta(seconds=60))
    peer = 1 - rank
    payload, inbox = torch.zeros(256), torch.zeros(256)
    record = {}

    def exchange(first: bool) -> None:
        if first:
            engine.submit(payload, peer, 1, True).wait(30)
            engine.submit(inbox, peer, 2, False).wait(30)
        else:
            engine.submit(inbox, peer, 1, False).wait(30)
            engine.submit(payload, peer, 2, True).wait(30)

    for _ in range(args.warmup):
        exchange(rank == 0)
    trips = []
    with Phase(store) as phase:
        for _ in range(args.iterations):
            t0 = time.perf_counter()
            exchange(rank == 0)
            trips.append(time.perf_counter() - t0)
    record["pingpong"] = dict(phase.result, one_way_us=round(statistics.median(trips) / 2 * 1e6, 1),
                              store_calls_per_message=round(sum(phase.result["store_calls"].values())
                                                            / (2 * args.iterations), 2))
    with Phase(store) as phase:
        time.sleep(args.idle)
    record["idle"] = phase.result
    with Phase(store) as phase:
        stuck = [engine.submit(payload, 1 - rank, 100 + i, True) for i in range(args.missing)] if rank == 0 else []
        t0 = time.perf_counter()
        exchange(rank == 0)
        live = time.perf_counter() - t0
        time.sleep(args.hold)
        t0 = time.perf_counter()
        engine.close()
        closed = time.perf_counter() - t0
    record["missing"] = dict(phase.result, live_exchange_us=round(live * 1e6, 1), close_ms=round(closed * 1e3, 2),
                             waiting=len(stuck))
    out.put((rank, record))


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    parser.add_argument("--store", choices=("tcp", "file"), default="file")
    parser.add_argument("--port", type=int, default=29641)
    parser.add_argument("--iterations", type=int, default=1000)
    parser.add_argument("--warmup", type=int, default=50)
    parser.add_argument("--idle", type=float, default=1.0)
    parser.add_argument("--missing", type=int, default=8)
    parser.add_argument("--hold", type=float, default=1.0)
    args = parser.parse_args(argv)
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    with tempfile.TemporaryDirectory() as scratch:
        procs = [ctx.Process(target=worker, args=(r, args, os.path.join(scratch, "store"), out)) for r in (0, 1)]
        [p.start() for p in procs]
        got = dict(out.get(timeout=300) for _ in procs)
        [p.join(30) for p in procs]
    print(json.dumps({"bench": "p2p_handshake", "store": args.store, "iterations": args.iterations,
                      "rank0": got[0], "rank1": got[1]}, indent=1))
    return 0


if __name__ == "__main__":
    sys.exit(main())
