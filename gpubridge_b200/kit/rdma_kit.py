"""Kit programs for the RDMA-style endpoint and the ``verbs`` bridge, over the in-process fabric.

    python -m gpubridge_b200.kit.rdma_kit check --out results/rdma      # protocol scenarios
    python -m gpubridge_b200.kit.rdma_kit perf  --out results/rdma      # size sweep
    python -m gpubridge_b200.kit.rdma_kit ab    --out results/rdma      # settings against each other

``check`` drives two to four members through what the wire protocol promises and writes one
row per scenario: eager and rendezvous messages arrive intact, a receive posted late finds its
message in the unexpected queue, a sender out of credits stalls and resumes, registrations are
cached and dropped on invalidate, tagged collectives give the known sums, and each injected
fault (an operation that fails, is dropped, delayed or corrupted; a member that dies) ends the
waits of everybody involved with an error inside the time limit and leaves the endpoints
broken; three more rows come from the registrar of device memory (which method it picks,
every reason when none works, a reused address as another owner).  ``perf`` times ping-pong latency and one-way bandwidth by message size.  ``ab`` runs
the bridge's all-reduce of one tensor under several settings (eager limit, write size, piece
size of the bounce path) and reports each against the first.  Numbers from the in-process
fabric measure this library's own work per message - queueing, matching, copying - not a
network (the reference's counterparts on real adapters: scripts/gpu/verbs_kit.py,
scripts/gpu/verbs_staged_ab.py, scripts/verbs_perf.py).
"""
from __future__ import annotations

import argparse
import json
import statistics
import sys
import threading
import time
from datetime import timedelta
from pathlib import Path

import torch

from gpubridge_b200 import rdma
from gpubridge_b200.rdma_transport import RdmaTransport


def _threads(count: int, body) -> list:
    out, errors = [None] * count, [None] * count

    def run(i: int) -> None:
        try:
            out[i] = body(i)
        except BaseException as failure:  # noqa: BLE001 - reported per member
            errors[i] = f"{type(failure).__name__}: {failure}"

    workers = [threading.Thread(target=run, args=(i,), daemon=True) for i in range(count)]
    for w in workers:
        w.start()
    for w in workers:
        w.join(60)
    return [{"value": o, "error": e} for o, e in zip(out, errors)]


# ---- check ------------------------------------------------------------------------------------------
def _exchange(nbytes: int, late_receive: bool = False, **settings) -> dict:
    fabric = rdma.MockFabric(2)
    ends = [fabric.endpoint(i, **settings) for i in range(2)]
    payload = torch.arange(nbytes, dtype=torch.uint8)
    landed = torch.zeros(nbytes, dtype=torch.uint8)

    def body(i: int):
        deadline = time.monotonic() + 10
        if i == 0:
            ends[0].wait([ends[0].send(1, payload.data_ptr(), nbytes, 7)], deadline)
        else:
            if late_receive:
                time.sleep(0.2)
            ends[1].wait([ends[1].recv(0, landed.data_ptr(), nbytes, 7)], deadline)
        return ends[i].telemetry()

    result = _threads(2, body)
    fabric.close()
    ok = all(r["error"] is None for r in result) and torch.equal(payload, landed)
    return {"ok": ok, "sender": result[0]["value"], "receiver": result[1]["value"],
            "errors": [r["error"] for r in result if r["error"]]}


def _fault(kind: str, members: int = 2) -> dict:
    fabric = rdma.MockFabric(members)
    bridges = [RdmaTransport.over_fabric(fabric, list(range(members)), m, timeout=timedelta(seconds=3))
               for m in range(members)]
    if kind == "kill":
        fabric.inject("kill", dst=members - 1, nth=2)
    else:
        fabric.inject(kind, src=0, dst=1, nth=2, milliseconds=4000 if kind == "delay" else 0)
    started = time.monotonic()
    result = _threads(members, lambda i: bridges[i].all_reduce(torch.ones(1 << 18)))
    took = time.monotonic() - started
    broken = [b.worker.telemetry()["broken"] for b in bridges]
    for b in bridges:
        b.close()
    fabric.close()
    failed = [r["error"] is not None for r in result]
    # a corrupted payload is caught by the sums check of the caller, not by the endpoint
    ok = (any(failed) and took < 10) if kind != "corrupt" else took < 10
    return {"ok": ok, "seconds": round(took, 2), "members_failed": failed, "broken": broken}


def _harmless(kind: str) -> dict:
    """Faults the protocol has to shrug off: the all-reduce still gives the known sum, nothing breaks."""
    fabric = rdma.MockFabric(2)
    bridges = [RdmaTransport.over_fabric(fabric, [0, 1], m, timeout=timedelta(seconds=10)) for m in (0, 1)]
    for nth in (1, 2, 4):
        fabric.inject(kind, src=0, dst=1, nth=nth, milliseconds=5 if kind == "spurious" else 150)

    def body(i: int):
        t = torch.arange(300_000, dtype=torch.float32) + i
        bridges[i].all_reduce(t)
        return bool(torch.equal(t, 2 * torch.arange(300_000, dtype=torch.float32) + 1))

    result = _threads(2, body)
    broken = [b.worker.telemetry()["broken"] for b in bridges]
    for b in bridges:
        b.close()
    fabric.close()
    return {"ok": all(r["value"] is True for r in result) and not any(broken), "broken": broken,
            "errors": [r["error"] for r in result if r["error"]]}


def _registration() -> list[tuple[str, dict]]:
    """The registrar of device memory on pretend device memory and a pretend adapter: the method
    it picks, what it says when no method works, and that a stale address is another owner."""
    import tempfile

    from gpubridge_b200 import rdma_direct
    found = []
    with tempfile.TemporaryDirectory() as root:
        Path(root, "proc").mkdir()
        Path(root, "proc", "modules").write_text("nvidia_peermem 16384 0 - Live 0x0\n")
        registrar = rdma_direct.Registrar.pretend(root)
        try:
            a = registrar.alloc(8 << 20)
            with registrar.acquire(a, 1 << 20) as first:
                pass
            registrar.invalidate(a, 8 << 20)
            registrar.fail("device dma-buf", "not exported")
            with registrar.acquire(a, 1 << 20) as second:
                pass
            found.append(("device registration: dma-buf first, then peer memory",
                          {"ok": (first.method, second.method) == ("dma-buf", "peer memory"),
                           "methods": [first.method, second.method]}))
            registrar.invalidate(a, 8 << 20)
            registrar.fail("device peer memory", "not allowed")
            try:
                registrar.take(a, 1 << 20)
                reasons = None
            except rdma_direct.NotDirect as why:
                reasons = str(why)
            found.append(("device registration: every reason when nothing works",
                          {"ok": reasons == "dma-buf: not exported; peer memory: not allowed", "reasons": reasons}))
            registrar.fail("device dma-buf")
            with registrar.acquire(a, 1 << 20) as old:
                pass
            registrar.free(a)
            registrar.alloc(8 << 20, at=a)
            with registrar.acquire(a, 1 << 20) as new:
                pass
            told = registrar.telemetry()
            found.append(("device registration: the same address later is another owner",
                          {"ok": new.key != old.key and told["stale_dropped"] == 1, "telemetry": told}))
        finally:
            registrar.close()
    return found


def check(out: Path) -> int:
    rows = []

    def row(name: str, result: dict) -> None:
        rows.append({"scenario": name, **result})
        print(f"[rdma-kit] {name}: {'ok' if result['ok'] else 'FAILED'}", flush=True)

    row("eager message", _exchange(2048))
    row("rendezvous message", _exchange(4 << 20))
    late = _exchange(2048, late_receive=True)
    late["ok"] = late["ok"] and late["receiver"]["unexpected"] >= 1
    row("receive posted late (unexpected queue)", late)
    stalled = _exchange(64 << 10, eager_max=1024, data_slots=2, max_write=4096)
    row("small windows (many writes)", dict(stalled, ok=stalled["ok"] and stalled["sender"]["writes"] > 4))
    for members in (2, 3, 4):
        fabric = rdma.MockFabric(members)
        bridges = [RdmaTransport.over_fabric(fabric, list(range(members)), m) for m in range(members)]

        def body(i, bridges=bridges, members=members):
            t = torch.arange(100_000, dtype=torch.float32) + i
            bridges[i].all_reduce(t)
            return bool(torch.equal(t, members * torch.arange(100_000, dtype=torch.float32)
                                    + sum(range(members))))

        result = _threads(members, body)
        for b in bridges:
            b.close()
        fabric.close()
        row(f"all-reduce of {members} members", {"ok": all(r["value"] is True for r in result),
                                                 "errors": [r["error"] for r in result if r["error"]]})
    for kind in ("error", "drop", "delay", "corrupt", "kill"):
        row(f"fault: {kind}", _fault(kind, 3 if kind == "kill" else 2))
    row("spurious wake-ups are harmless", _harmless("spurious"))
    row("a completion that comes after the peer's answer is harmless", _harmless("late"))
    for name, result in _registration():
        row(name, result)
    out.mkdir(parents=True, exist_ok=True)
    (out / "rdma_check.json").write_text(json.dumps({"schema": "gpubridge_b200.rdma_kit/1", "rows": rows}, indent=1))
    failed = [r["scenario"] for r in rows if not r["ok"]]
    print("every scenario passed" if not failed else f"failed: {', '.join(failed)}")
    return 1 if failed else 0


# ---- perf -------------------------------------------------------------------------------------------
def _socket_pair() -> list:
    """Two endpoints joined by the Unix-domain socket provider, made in two threads."""
    names, ready, ends = [None, None], threading.Barrier(2), [None, None]

    def make(i: int) -> None:
        def publish(name: str) -> None:
            names[i] = name
            ready.wait(20)
        ends[i] = rdma.Endpoint.over_sockets(i, 2, publish, lambda: list(names), 20.0)

    workers = [threading.Thread(target=make, args=(i,)) for i in range(2)]
    for w in workers:
        w.start()
    for w in workers:
        w.join(30)
    if None in ends:
        raise RuntimeError("the socket provider did not connect")
    return ends


def perf(out: Path, sizes: list[int], trials: int, fabric_kind: str = "memory") -> int:
    rows = []
    for nbytes in sizes:
        if fabric_kind == "sockets":
            fabric, ends = None, _socket_pair()
        else:
            fabric = rdma.MockFabric(2)
            ends = [fabric.endpoint(i) for i in range(2)]
        # every member has its own pair of buffers (real pages, not the zero page)
        pairs = [[torch.randint(0, 255, (nbytes,), dtype=torch.uint8) for _ in range(2)] for _ in range(2)]
        laps: list[float] = []

        def body(i: int, ends=ends, pairs=pairs, laps=laps, nbytes=nbytes):
            deadline = time.monotonic() + 60
            there, back = pairs[i]
            for lap in range(trials + 2):
                t0 = time.perf_counter()
                if i == 0:
                    ends[0].wait([ends[0].send(1, there.data_ptr(), nbytes, lap)], deadline)
                    ends[0].wait([ends[0].recv(1, back.data_ptr(), nbytes, lap)], deadline)
                    if lap >= 2:
                        laps.append(time.perf_counter() - t0)
                else:
                    ends[1].wait([ends[1].recv(0, there.data_ptr(), nbytes, lap)], deadline)
                    ends[1].wait([ends[1].send(0, back.data_ptr(), nbytes, lap)], deadline)

        result = _threads(2, body)
        if fabric is not None:
            fabric.close()
        else:
            closers = [threading.Thread(target=e.close) for e in ends]      # they say goodbye to each other
            for c in closers:
                c.start()
            for c in closers:
                c.join(15)
        if any(r["error"] for r in result) or not laps:
            rows.append({"bytes": nbytes, "error": [r["error"] for r in result if r["error"]]})
            continue
        half = statistics.median(laps) / 2
        rows.append({"bytes": nbytes, "fabric": fabric_kind, "one_way_us": round(half * 1e6, 1),
                     "gbs": round(nbytes / half / 1e9, 3)})
        print(json.dumps(rows[-1]), flush=True)
    out.mkdir(parents=True, exist_ok=True)
    (out / "rdma_perf.json").write_text(json.dumps({"schema": "gpubridge_b200.rdma_kit/1", "rows": rows}, indent=1))
    return 1 if any("error" in r for r in rows) else 0


# ---- ab ---------------------------------------------------------------------------------------------
ARMS = [("defaults", {}), ("eager up to 64 KiB", {"eager_max": 64 << 10}),
        ("writes of 256 KiB", {"max_write": 256 << 10}), ("pieces of 1 MiB", {"piece_bytes": 1 << 20}),
        ("pieces of 32 MiB", {"piece_bytes": 32 << 20})]


def ab(out: Path, numel: int, trials: int) -> int:
    rows = []
    for label, settings in ARMS:
        fabric = rdma.MockFabric(2)
        bridges = [RdmaTransport.over_fabric(fabric, [0, 1], m, **settings) for m in (0, 1)]
        tensors = [torch.ones(64, numel // 64).t() for _ in (0, 1)]        # strided: the bounce path
        laps: list[float] = []

        def body(i: int, bridges=bridges, tensors=tensors, laps=laps):
            for lap in range(trials + 1):
                t0 = time.perf_counter()
                bridges[i].all_reduce(tensors[i])
                if i == 0 and lap:
                    laps.append(time.perf_counter() - t0)

        result = _threads(2, body)
        described = bridges[0].describe()
        for b in bridges:
            b.close()
        fabric.close()
        if any(r["error"] for r in result):
            rows.append({"arm": label, "error": [r["error"] for r in result if r["error"]]})
            continue
        rows.append({"arm": label, "settings": settings, "ms": round(statistics.median(laps) * 1e3, 3),
                     "routes": described["routes"], "staging": described["staging"]})
    base = next((r["ms"] for r in rows if "ms" in r), None)
    for r in rows:
        if "ms" in r and base:
            r["against_first"] = round(r["ms"] / base, 3)
        print(json.dumps(r), flush=True)
    out.mkdir(parents=True, exist_ok=True)
    (out / "rdma_ab.json").write_text(json.dumps({"schema": "gpubridge_b200.rdma_kit/1", "numel": numel,
                                                   "rows": rows}, indent=1))
    return 1 if any("error" in r for r in rows) else 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("what", choices=("check", "perf", "ab"))
    ap.add_argument("--out", type=Path, required=True)
    ap.add_argument("--trials", type=int, default=20)
    ap.add_argument("--sizes", default="64,4096,65536,1048576,16777216")
    ap.add_argument("--numel", type=int, default=1 << 22)
    ap.add_argument("--fabric", default="memory", choices=("memory", "sockets"),
                    help="perf: the in-process fabric, or the Unix-domain socket provider")
    args = ap.parse_args(argv)
    if args.what == "check":
        return check(args.out)
    if args.what == "perf":
        return perf(args.out, [int(s) for s in args.sizes.split(",")], args.trials, args.fabric)
    return ab(args.out, args.numel, args.trials)


if __name__ == "__main__":
    sys.exit(main())
