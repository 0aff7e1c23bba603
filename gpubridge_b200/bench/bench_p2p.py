"""Point-to-point latency and bandwidth through ``backend="gpubridge"``, per route.

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 \
        -m gpubridge_b200.bench.bench_p2p --out results/p2p
    GPUBRIDGE_VENDOR=nvidia GPUBRIDGE_SPLIT_TEST=half python -m torch.distributed.run \
        --nproc-per-node 4 --master-addr 127.0.0.1 -m gpubridge_b200.bench.bench_p2p \
        --out /tmp/p2p --max-bytes 4M                                  # CPU simulation

Rank 0 plays ping-pong with one peer per route while the other ranks wait at a barrier:
``bridge`` = the lowest rank of another island, ``native`` = the next rank of rank 0's own
island.  On one NVSwitch box both go over NCCL send/recv (every GPU reaches every other); in
simulation and across hosts the bridge route is the host-staged engine.  Every size starts
with an untimed exchange whose payload is checked bit for bit in both directions; then
``--warmup`` untimed and ``--trials`` timed round trips.  One-way latency is half the median
round trip (host clock, device synchronised on both sides), bandwidth is bytes over that.
Rank 0 writes ``bench_p2p.json`` and ``summary.md``.  Same measurement as the reference's
``scripts/gpu/bench_p2p.py`` (:78-116).
"""
from __future__ import annotations

import argparse
import statistics
import sys
import time
from datetime import timedelta
from pathlib import Path

import torch
import torch.distributed as dist

import gpubridge_b200 as gb
from gpubridge_b200.config import parse_size
from gpubridge_b200.kit import default_timeout, environment, run_info, sync, write_json

TAG = 7


def routes(topology) -> dict[str, int]:
    layout = topology.layout
    own = layout.island_of(0)
    found: dict[str, int] = {}
    others = [i for i in layout.islands if i != own]
    if others:
        found["bridge"] = min(others[0].ranks)
    if len(own.ranks) > 1:
        found["native"] = sorted(own.ranks)[1]
    return found


def pattern(numel: int, device: torch.device) -> torch.Tensor:
    """Integer-valued float32s, distinct modulo 251, built in bounded pieces."""
    out = torch.empty(numel, dtype=torch.float32, device=device)
    step = 1 << 20
    for lo in range(0, numel, step):
        n = min(step, numel - lo)
        out[lo:lo + n].copy_(torch.arange(lo % 251, lo % 251 + n, dtype=torch.int64).remainder_(251).float())
    return out


def ping(peer: int, numel: int, device, warmup: int, trials: int):
    sent = pattern(numel, device)
    back = torch.full_like(sent, -1)
    dist.send(sent, peer, tag=TAG)
    dist.recv(back, peer, tag=TAG)
    sync(device)
    intact = bool(torch.equal(back, sent))
    times = []
    for i in range(warmup + trials):
        sync(device)
        t0 = time.perf_counter()
        dist.send(sent, peer, tag=TAG)
        dist.recv(back, peer, tag=TAG)
        sync(device)
        if i >= warmup:
            times.append(time.perf_counter() - t0)
    return times, intact


def pong(numel: int, device, rounds: int) -> bool:
    buf = torch.empty(numel, dtype=torch.float32, device=device)
    dist.recv(buf, 0, tag=TAG)
    intact = bool(torch.equal(buf, pattern(numel, device)))
    dist.send(buf, 0, tag=TAG)
    for _ in range(rounds):
        dist.recv(buf, 0, tag=TAG)
        dist.send(buf, 0, tag=TAG)
    return intact


def human(n: int) -> str:
    for unit, size in (("G", 1 << 30), ("M", 1 << 20), ("K", 1 << 10)):
        if n >= size and n % size == 0:
            return f"{n // size}{unit}"
    return str(n)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--out", type=Path, required=True)
    ap.add_argument("--min-bytes", type=parse_size, default=parse_size("1K"))
    ap.add_argument("--max-bytes", type=parse_size, default=parse_size("1G"))
    ap.add_argument("--factor", type=int, default=4)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--trials", type=int, default=10)
    ap.add_argument("--timeout", type=float, default=default_timeout(600))
    args = ap.parse_args(argv)
    if args.factor <= 1 or args.min_bytes <= 0 or args.max_bytes < args.min_bytes:
        ap.error("need --factor > 1 and 0 < --min-bytes <= --max-bytes")
    if args.trials <= 0 or args.warmup < 0:
        ap.error("--trials must be positive and --warmup nonnegative")
    dist.init_process_group("gpubridge", timeout=timedelta(seconds=args.timeout))
    dist.barrier()
    topology = gb.get_topology()
    rank, device = topology.rank, topology.device
    if topology.world_size < 2:
        raise SystemExit("bench_p2p needs at least two ranks")
    rows = []
    nbytes = args.min_bytes
    sizes = []
    while nbytes <= args.max_bytes:
        sizes.append(nbytes)
        nbytes *= args.factor
    for route, peer in routes(topology).items():
        for size in sizes:
            numel = max(1, size // 4)
            if rank == 0:
                times, intact = ping(peer, numel, device, args.warmup, args.trials)
                rtt = statistics.median(times)
                ordered = sorted(times)
                rows.append({"route": route, "peer": peer, "bytes": numel * 4,
                             "one_way_us": round(rtt / 2 * 1e6, 2),
                             "bandwidth_GBps": round(numel * 4 / (rtt / 2) / 1e9, 3),
                             "rtt_p90_us": round(ordered[min(len(ordered) - 1, int(0.9 * len(ordered)))] * 1e6, 2),
                             "payload_ok": intact})
            elif rank == peer:
                if not pong(numel, device, args.warmup + args.trials):
                    raise AssertionError(f"rank {rank}: payload of {numel * 4} bytes arrived damaged")
            dist.barrier()
    ok = all(r["payload_ok"] for r in rows)
    if rank == 0:
        record = {"environment": environment(), "run": run_info(topology), "rows": rows, "ok": ok}
        write_json(args.out / "bench_p2p.json", record)
        lines = ["Ping-pong between rank 0 and each route's peer; one-way = half the median round trip.",
                 "", "| route | peer | size | one-way (us) | GB/s | round trip p90 (us) | payload |",
                 "| --- | ---: | --- | ---: | ---: | ---: | --- |"]
        for r in rows:
            lines.append(f"| {r['route']} | {r['peer']} | {human(r['bytes'])} | {r['one_way_us']} | "
                         f"{r['bandwidth_GBps']} | {r['rtt_p90_us']} | {'ok' if r['payload_ok'] else 'WRONG'} |")
        (args.out / "summary.md").write_text("\n".join(lines) + "\n")
        print("\n".join(lines))
    dist.destroy_process_group()
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
