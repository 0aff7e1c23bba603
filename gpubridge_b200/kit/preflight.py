"""Network preflight between two machines, for the host-staged bridge that joins boxes.

One NVSwitch box needs none of this (its GPUs talk over NVLink from inside the kernels); a job
that spans boxes joins them with a host bridge (``bridge="gloo"`` or ``"multitcp"``), and that
bridge is only as good as the interface it runs on.  Run on both machines at about the same
time, before the job:

    python -m gpubridge_b200.kit.preflight --role master --master-addr 10.0.0.1 --port 29501
    python -m gpubridge_b200.kit.preflight --role worker --master-addr 10.0.0.1 --port 29501

Steps: the master address resolves; both sides meet in a TCP store; each side lists its
candidate interfaces (IPv4, not loopback or link-local unless nothing else exists, or just
``--ifname`` / ``GLOO_SOCKET_IFNAME``); for every pair of addresses a connection each way,
the round-trip time (median of 50 one-byte ping-pongs) and the bandwidth each way for
``--bandwidth-seconds`` over one stream; the pair whose slower direction is fastest is chosen;
a real two-rank Gloo group on the chosen interfaces runs a barrier and an all-reduce (Gloo
connects on other ports, so this catches firewalls that only let the rendezvous through).
Exit code 0 on success; ``--out DIR`` gets ``preflight-<role>.json`` with ``chosen_ifname`` and
``chosen_address`` (use them as ``GLOO_SOCKET_IFNAME`` and ``GPUBRIDGE_MULTITCP_IFADDR``).
One Python-driven TCP stream understates fast links: read the bandwidth as a lower bound.
Counterpart of the reference's ``scripts/gpu/preflight.py``.
"""
from __future__ import annotations

import argparse
import json
import os
import socket
import statistics
import sys
import time
from datetime import timedelta
from pathlib import Path

NOTE = "raw TCP, one stream driven from Python: a lower bound on fast links"


def candidates(ifname: str | None) -> list[dict]:
    """[{ifname, address}] of this machine's usable IPv4 interfaces."""
    import psutil
    found, fallback = [], []
    for name, addresses in psutil.net_if_addrs().items():
        if ifname and name != ifname:
            continue
        for a in addresses:
            if a.family != socket.AF_INET:
                continue
            entry = {"ifname": name, "address": a.address}
            if a.address.startswith("127.") or a.address.startswith("169.254."):
                fallback.append(entry)
            else:
                found.append(entry)
    return found or fallback


def _serve(listener: socket.socket, seconds: float) -> None:
    """Echo the ping-pongs, then sink bytes for `seconds`, then source them."""
    conn, _ = listener.accept()
    with conn:
        conn.setsockopt(socket.IPPROTO_TCP, socket.TCP_NODELAY, 1)
        for _ in range(50):
            conn.sendall(conn.recv(1))
        _sink(conn)
        _source(conn, seconds)


def _sink(conn: socket.socket) -> int:
    total = 0
    while True:
        data = conn.recv(1 << 20)
        if not data or data.endswith(b"\xff"):
            return total + len(data)
        total += len(data)


def _source(conn: socket.socket, seconds: float) -> float:
    block = bytes(1 << 20)
    sent, t0 = 0, time.perf_counter()
    while time.perf_counter() - t0 < seconds:
        conn.sendall(block)
        sent += len(block)
    conn.sendall(b"\xff")
    return sent / (time.perf_counter() - t0) / 1e6


def _measure(address: str, port: int, bind: str, seconds: float) -> dict:
    with socket.create_connection((address, port), timeout=10, source_address=(bind, 0)) as conn:
        conn.setsockopt(socket.IPPROTO_TCP, socket.TCP_NODELAY, 1)
        trips = []
        for _ in range(50):
            t0 = time.perf_counter()
            conn.sendall(b"x")
            conn.recv(1)
            trips.append(time.perf_counter() - t0)
        out_mbs = _source(conn, seconds)
        t0 = time.perf_counter()
        received = _sink(conn)
        in_mbs = received / max(time.perf_counter() - t0, 1e-9) / 1e6
    return {"rtt_us": round(statistics.median(trips) * 1e6, 1), "out_MBps": round(out_mbs, 1),
            "in_MBps": round(in_mbs, 1), "note": NOTE}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--role", choices=("master", "worker", "auto"), default="auto")
    ap.add_argument("--master-addr", default=os.environ.get("MASTER_ADDR", "127.0.0.1"))
    ap.add_argument("--port", type=int, default=29501)
    ap.add_argument("--ifname", default=os.environ.get("GLOO_SOCKET_IFNAME") or None)
    ap.add_argument("--bandwidth-seconds", type=float, default=2.0)
    ap.add_argument("--timeout", type=float, default=120)
    ap.add_argument("--out", type=Path)
    args = ap.parse_args(argv)
    role = args.role
    if role == "auto":
        role = "master" if int(os.environ.get("SLURM_PROCID", os.environ.get("RANK", "0"))) == 0 else "worker"
    master = role == "master"
    record: dict = {"role": role, "hostname": socket.gethostname(), "checks": {}, "ok": False}

    def finish(code: int) -> int:
        record["ok"] = code == 0
        if args.out:
            args.out.mkdir(parents=True, exist_ok=True)
            (args.out / f"preflight-{role}.json").write_text(json.dumps(record, indent=1))
        print(json.dumps({k: record[k] for k in ("role", "ok", "chosen_ifname", "chosen_address")
                          if k in record}))
        return code

    try:
        record["checks"]["resolve"] = socket.gethostbyname(args.master_addr)
    except OSError as exc:
        record["checks"]["resolve"] = f"failed: {exc}"
        return finish(1)
    mine = candidates(args.ifname)
    record["checks"]["interfaces"] = mine
    if not mine:
        return finish(1)
    from torch.distributed import TCPStore
    store = TCPStore(args.master_addr, args.port, 2, master, timedelta(seconds=args.timeout))
    record["checks"]["store"] = "ok"
    side, other = ("m", "w") if master else ("w", "m")
    # every candidate gets a listener; the other side connects to each from each of its own
    listeners = []
    for entry in mine:
        s = socket.socket(socket.AF_INET, socket.SOCK_STREAM)
        s.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
        s.bind((entry["address"], 0))
        s.listen(8)
        entry["port"] = s.getsockname()[1]
        listeners.append(s)
    store.set(f"pf/{side}/interfaces", json.dumps(mine))
    theirs = json.loads(store.get(f"pf/{other}/interfaces"))
    pairs = []
    # the worker measures towards the master first, then the master towards the worker
    for turn in ("w", "m"):
        if turn == side:
            for me in mine:
                for peer in theirs:
                    key = f"pf/go/{turn}/{me['address']}/{peer['address']}"
                    store.set(key, "1")
                    try:
                        numbers = _measure(peer["address"], peer["port"], me["address"],
                                           args.bandwidth_seconds)
                        pairs.append({"from": me, "to": peer, **numbers})
                    except OSError as exc:
                        pairs.append({"from": me, "to": peer, "error": str(exc)})
                        store.set(key + "/failed", "1")
            store.set(f"pf/done/{turn}", "1")
        else:
            import threading
            stop = threading.Event()

            def serve(listener):
                listener.settimeout(0.5)
                while not stop.is_set():
                    try:
                        _serve(listener, args.bandwidth_seconds)
                    except (TimeoutError, socket.timeout, OSError):
                        continue
            threads = [threading.Thread(target=serve, args=(s,), daemon=True) for s in listeners]
            [t.start() for t in threads]
            store.wait([f"pf/done/{turn}"], timedelta(seconds=args.timeout * 4))
            stop.set()
            [t.join(timeout=2) for t in threads]
    for s in listeners:
        s.close()
    record["checks"]["reachability"] = pairs
    store.set(f"pf/{side}/pairs", json.dumps(pairs))
    other_pairs = json.loads(store.get(f"pf/{other}/pairs"))
    # choose: both directions measured; maximise the slower direction
    best, best_rate = None, -1.0
    for p in pairs:
        if "error" in p:
            continue
        back = next((q for q in other_pairs if "error" not in q
                     and q["from"]["address"] == p["to"]["address"]
                     and q["to"]["address"] == p["from"]["address"]), None)
        if back is None:
            continue
        rate = min(p["out_MBps"], p["in_MBps"], back["out_MBps"], back["in_MBps"])
        if rate > best_rate:
            best, best_rate = p, rate
    if best is None:
        record["checks"]["choose"] = "no pair of interfaces connects both ways"
        return finish(1)
    record["chosen_ifname"] = best["from"]["ifname"]
    record["chosen_address"] = best["from"]["address"]
    record["bandwidth"] = {k: best[k] for k in ("rtt_us", "out_MBps", "in_MBps", "note")}
    # a real Gloo pair on the chosen interfaces
    import torch
    import torch.distributed as dist
    os.environ["GLOO_SOCKET_IFNAME"] = record["chosen_ifname"]
    try:
        dist.init_process_group("gloo", store=store, rank=0 if master else 1, world_size=2,
                                timeout=timedelta(seconds=args.timeout))
        dist.barrier()
        t = torch.ones(1024)
        dist.all_reduce(t)
        record["checks"]["gloo"] = "ok" if bool((t == 2).all()) else "wrong result"
        dist.destroy_process_group()
    except Exception as exc:  # noqa: BLE001
        record["checks"]["gloo"] = f"failed: {type(exc).__name__}: {exc}"
        return finish(1)
    return finish(0 if record["checks"]["gloo"] == "ok" else 1)


if __name__ == "__main__":
    sys.exit(main())
