"""Per-rank correctness check, launched by torchrun; one JSON journal per rank.

    torchrun --nproc-per-node 8 -m gpubridge_b200.kit.check --out results/check8
    GPUBRIDGE_ISLANDS=4,4 torchrun --nproc-per-node 8 -m gpubridge_b200.kit.check --out ...
    python -m gpubridge_b200.kit.summarize results/check8

The same thirteen stages as the reference's ``scripts/gpu/check.py`` (stage list :6-27, main
:103-271): init, device, dtypes, busy_gpu, broadcast, reductions, all_gather, reduce_scatter,
async, reduction_agreement, in_flight, barrier, destroy.  Every check uses small integers
that differ per rank and element, so any summation order gives the same exact answer.

``--expect-init-error REGEX`` makes the run a negative test: ``init()`` must fail on every
rank with a matching message (check.py:407-429 there).  ``--p2p-only`` initialises the torch
backend instead and runs the point-to-point checks.
"""
from __future__ import annotations

import argparse
import os
import re
import sys
import threading
import time
import traceback
from datetime import timedelta
from pathlib import Path

import torch

import gpubridge_b200 as gb
from gpubridge_b200.collectives import SUPPORTED_DTYPES
from gpubridge_b200.kit import (Journal, default_timeout, queue_gpu_delay, rank_from_env,
                                run_info, sync)

DTYPES = {str(d).removeprefix("torch."): d for d in SUPPORTED_DTYPES}
#: What the busy-GPU and async tensors hold until the queued work ahead of them is done.
POISON = -1000.0
OPS = {"sum": gb.ReduceOp.SUM, "avg": gb.ReduceOp.AVG, "max": gb.ReduceOp.MAX,
       "min": gb.ReduceOp.MIN}


def _pattern(shape, dtype: torch.dtype, rank: int) -> torch.Tensor:
    """float64 values: at most 16 per element (exact in bf16 for 16 ranks), at most 3 for
    8-bit types."""
    n = int(torch.Size(shape).numel())
    idx = torch.arange(n, dtype=torch.float64).reshape(shape)
    if dtype in (torch.int8, torch.uint8):
        return idx % 2 + rank % 2 + 1
    return idx % 8 + rank % 8 + 1


def values(shape, dtype, rank, device) -> torch.Tensor:
    return _pattern(shape, dtype, rank).to(dtype).to(device)


def reduced(shape, dtype, world, device, op: str) -> torch.Tensor:
    stack = torch.stack([_pattern(shape, dtype, r) for r in range(world)])
    if op in ("sum", "avg"):
        out = stack.sum(0).to(dtype)
        return (out.div(world) if op == "avg" else out).to(device)
    return (stack.amax(0) if op == "max" else stack.amin(0)).to(dtype).to(device)


def differ(got: torch.Tensor, want: torch.Tensor) -> dict | None:
    if torch.equal(got, want):
        return None
    delta = (got.double() - want.double()).abs()
    return {"max_abs_error": float(delta.max()), "wrong_elements": int((delta > 0).sum())}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--out", type=Path, required=True)
    ap.add_argument("--timeout", type=float, default=default_timeout(600))
    ap.add_argument("--dtypes", default=",".join(DTYPES))
    ap.add_argument("--policy", default="auto")
    ap.add_argument("--bridge", default=os.environ.get("GPUBRIDGE_BRIDGE", "").strip() or None,
                    help="bridge transport (default: GPUBRIDGE_BRIDGE, else init()'s choice)")
    ap.add_argument("--p2p-only", action="store_true")
    ap.add_argument("--large-numel", type=int, default=None)
    ap.add_argument("--busy-seconds", type=float, default=0.05)
    ap.add_argument("--in-flight-settle", type=float, default=1.0)
    ap.add_argument("--expect-init-error", metavar="REGEX")
    args = ap.parse_args(argv)

    rank = rank_from_env()
    journal = Journal(args.out / f"rank{rank}.json", "gpubridge_b200.kit.check",
                      hang_dump_seconds=args.timeout * 0.8)
    if args.expect_init_error:
        return _expect_init_error(journal, args)
    if args.p2p_only:
        return _p2p_only(journal, args)
    init_kwargs = {"timeout": timedelta(seconds=args.timeout), "policy": args.policy}
    if args.bridge:
        init_kwargs["bridge"] = args.bridge
    try:
        with journal.stage("init"):
            topology = gb.init(**init_kwargs)
        journal.data["run"] = run_info(topology)
        journal.flush()
        if topology.split_test and rank == 0:
            print(journal.data["run"]["warning"], file=sys.stderr, flush=True)
        device, world = topology.device, topology.world_size
        names = [n for n in args.dtypes.split(",") if n]

        with journal.stage("device") as e:
            e["device"] = str(device)
            if device.type == "cuda":
                index = torch.cuda.current_device()
                props = torch.cuda.get_device_properties(index)
                e.update(current_device=index, name=props.name,
                         uuid=str(getattr(props, "uuid", "")) or None)
                e["ok"] = index == device.index

        with journal.stage("dtypes") as e:
            e["cases"] = []
            for name in names:
                t = values((1024, 3), DTYPES[name], rank, device)
                gb.all_reduce(t)
                bad = differ(t, reduced((1024, 3), DTYPES[name], world, device, "sum"))
                e["cases"].append({"dtype": name, "ok": bad is None, **(bad or {})})
            e["ok"] = all(c["ok"] for c in e["cases"])

        with journal.stage("busy_gpu") as e:
            numel = args.large_numel or ((64 << 20) if device.type == "cuda" else (1 << 20))
            e["numel"], e["megabytes"] = numel, round(numel * 4 / 2**20, 1)
            t = torch.full((numel,), float(rank + 1), device=device)
            if device.type == "cuda":
                # the tensor holds poison until work queued ahead of the collective is done;
                # a collective that did not wait for the stream would reduce the poison
                t.fill_(POISON)
                queue_gpu_delay(device, args.busy_seconds)
                t.fill_(float(rank + 1))
            t0 = time.perf_counter()
            gb.all_reduce(t)
            sync(device)
            e["all_reduce_seconds"] = round(time.perf_counter() - t0, 4)
            want = world * (world + 1) / 2
            e["ok"] = bool(torch.all(t == want))
            if not e["ok"]:
                e["wrong_elements"] = int((t != want).sum())

        with journal.stage("broadcast") as e:
            e["bad_sources"] = []
            for src in range(world):
                t = values((257,), torch.float32, rank, device)
                gb.broadcast(t, src)
                if not torch.equal(t, values((257,), torch.float32, src, device)):
                    e["bad_sources"].append(src)
            e["ok"] = not e["bad_sources"]

        with journal.stage("reductions") as e:
            e["cases"] = []
            for name in names:
                dtype = DTYPES[name]
                for op in ("max", "min") + (("avg",) if dtype.is_floating_point else ()):
                    t = values((1024, 3), dtype, rank, device)
                    gb.all_reduce(t, op=OPS[op])
                    bad = differ(t, reduced((1024, 3), dtype, world, device, op))
                    e["cases"].append({"dtype": name, "op": op, "ok": bad is None, **(bad or {})})
            e["ok"] = all(c["ok"] for c in e["cases"])

        with journal.stage("all_gather") as e:
            e["cases"] = []
            for name in names:
                dtype = DTYPES[name]
                out = torch.empty((world * 257, 2), dtype=dtype, device=device)
                gb.all_gather_into_tensor(out, values((257, 2), dtype, rank, device))
                want = torch.cat([values((257, 2), dtype, r, device) for r in range(world)])
                bad = differ(out, want)
                e["cases"].append({"dtype": name, "ok": bad is None, **(bad or {})})
            e["ok"] = all(c["ok"] for c in e["cases"])

        with journal.stage("reduce_scatter") as e:
            e["cases"] = []
            for name in names:
                dtype = DTYPES[name]
                for op in ("sum",) + (("avg",) if dtype.is_floating_point else ()):
                    out = torch.empty(129, dtype=dtype, device=device)
                    gb.reduce_scatter_tensor(out, values((world * 129,), dtype, rank, device),
                                             op=OPS[op])
                    want = reduced((world * 129,), dtype, world, device, op)
                    bad = differ(out, want[rank * 129:(rank + 1) * 129])
                    e["cases"].append({"dtype": name, "op": op, "ok": bad is None, **(bad or {})})
            e["ok"] = all(c["ok"] for c in e["cases"])

        with journal.stage("async") as e:
            numel = (4 << 20) if device.type == "cuda" else (1 << 16)
            t = torch.full((numel,), float(rank + 1), device=device)
            if device.type == "cuda":
                t.fill_(POISON)
                queue_gpu_delay(device, args.busy_seconds)
                t.fill_(float(rank + 1))
            work = gb.all_reduce(t, async_op=True)
            work.wait()                       # orders this stream; the host does not block
            right = t == world * (world + 1) / 2
            e["ok"] = bool(right.all())
            e["is_completed"] = work.is_completed()
            if not e["ok"]:
                e["wrong_elements"] = int((~right).sum())

        with journal.stage("reduction_agreement") as e:
            e.update(_reduction_agreement(topology))

        with journal.stage("in_flight") as e:
            e.update(_late_rank_view(topology, args.in_flight_settle, args.timeout))

        with journal.stage("barrier"):
            gb.barrier()
            sync(device)

        with journal.stage("destroy") as e:
            describe = getattr(topology.bridge, "describe", None)
            if describe is not None:               # a leader whose bridge keeps counts: routes, staging, counters
                try:
                    e["bridge"] = describe()
                except Exception as failure:  # noqa: BLE001 - a record less, never a failed stage
                    e["bridge"] = f"no report: {type(failure).__name__}: {failure}"
            gb.destroy()
    except BaseException:
        traceback.print_exc()
        journal.failed = True
    return journal.close()


def _reduction_agreement(topology) -> dict:
    """Informational: what MAX and MIN do with a NaN on one rank, in the path a user calls
    and on the host (Gloo) communicator.  The fused kernels fold with fmax / fmin, which
    drop a NaN; host libraries differ among themselves.  PRODUCT is not offered by any
    policy here (the reference's bridged policies refuse it too)."""
    rank, device = topology.rank, topology.device
    host = topology.cpu_group
    answers = {}
    for name, dtype in DTYPES.items():
        if not dtype.is_floating_point:
            continue
        v = torch.tensor([1.0, -2.0, 3.0]).to(dtype)
        if rank == topology.island.leader:
            v[0] = float("nan")
        for op in ("max", "min"):
            entry = {}
            try:
                mine = v.to(device)
                gb.all_reduce(mine, op=OPS[op])
                entry["ours_first"] = str(mine[0].item())
            except Exception as exc:
                entry["ours_error"] = type(exc).__name__
            if host is not None:
                try:
                    theirs = v.clone()
                    host.all_reduce(theirs, op)
                    entry["host_first"] = str(theirs[0].item())
                except Exception as exc:
                    entry["host_error"] = type(exc).__name__
            entry["agree"] = entry.get("ours_first") == entry.get("host_first")
            answers[f"{name}/{op}"] = entry
    return {"ok": True, "product": "not offered", "nan_max_min": answers}


def _late_rank_view(topology, settle: float, timeout: float) -> dict:
    """The last rank joins an all-reduce only after every other rank's ``in_flight()`` view,
    sampled from a second thread, has stopped changing; the order is kept through the job's
    store, not by sleeping.  The late rank must show nothing in flight before it joins and
    every entry anywhere must be this all-reduce."""
    rank, world, device = topology.rank, topology.world_size, topology.device
    store = topology.context.store
    late = world - 1
    key = f"kit-check/in_flight/{os.environ.get('TORCHELASTIC_RESTART_COUNT', '0')}"
    t = torch.ones(16, device=device)
    seen: list[list] = []
    if world == 1:
        gb.all_reduce(t)
        return {"late_rank": 0, "in_flight": [], "ok": True}
    if rank == late:
        deadline = time.monotonic() + timeout
        keys = [f"{key}/settled/{r}" for r in range(late)]
        while not store.check(keys):
            if time.monotonic() > deadline:
                raise TimeoutError("the other ranks' in_flight() views did not settle")
            time.sleep(0.01)
        store.set(f"{key}/stop", "1")
        store.wait([f"{key}/done/{r}" for r in range(late)], timedelta(seconds=timeout))
        thread = threading.Thread(target=lambda: seen.append(gb.in_flight()))
        thread.start()
        thread.join()
        gb.all_reduce(t)
    else:
        returned = threading.Event()

        def watch() -> None:
            view, since, settled = None, time.monotonic(), False
            while not store.check([f"{key}/stop"]):
                flights = gb.in_flight()
                now = time.monotonic()
                current = [(f.seq, f.op, f.phase, tuple(f.phases_done)) for f in flights]
                if current != view:
                    view, since = current, now
                    if settled:
                        store.delete_key(f"{key}/settled/{rank}")
                        settled = False
                elif not settled and now - since >= settle and (flights or returned.is_set()):
                    store.set(f"{key}/settled/{rank}", "1")
                    settled = True
                time.sleep(0.01)
            seen.append(gb.in_flight())
            store.set(f"{key}/done/{rank}", "1")

        thread = threading.Thread(target=watch, daemon=True)
        thread.start()
        gb.all_reduce(t)                 # fused: returns once the launch is queued
        returned.set()
        thread.join()
    sync(device)
    flights = [{"seq": f.seq, "op": f.op, "policy": f.policy, "phase": f.phase,
                "phases_done": list(f.phases_done), "seconds": round(f.seconds, 3)}
               for f in (seen[0] if seen else [])]
    ok = bool(seen) and all(f["op"] == "all_reduce" for f in flights)
    return {"late_rank": late, "settle_seconds": settle, "in_flight": flights,
            "ok": ok and (rank != late or not flights)}


def _expect_init_error(journal: Journal, args) -> int:
    with journal.stage("expected_init_error") as e:
        e["pattern"] = args.expect_init_error
        try:
            gb.init(timeout=timedelta(seconds=args.timeout), policy=args.policy)
        except RuntimeError as exc:
            print(f"rank {rank_from_env()}: init() failed: {exc}", file=sys.stderr, flush=True)
            e["message"] = str(exc)
            e["ok"] = re.search(args.expect_init_error, str(exc)) is not None
            if not e["ok"]:
                e["error"] = f"init() failed, but not with {args.expect_init_error!r}"
        else:
            gb.destroy()
            e["ok"] = False
            e["error"] = "init() succeeded; this run expected it to fail"
    return journal.close()


def _p2p_only(journal: Journal, args) -> int:
    import torch.distributed as dist
    from gpubridge_b200.kit.p2p_checks import p2p_checks
    if args.bridge:
        os.environ["GPUBRIDGE_BRIDGE"] = args.bridge
    os.environ["GPUBRIDGE_POLICY"] = args.policy
    try:
        with journal.stage("init"):
            dist.init_process_group("gpubridge", timeout=timedelta(seconds=args.timeout))
            dist.barrier()
        topology = gb.get_topology()
        journal.data["run"] = run_info(topology)
        with journal.stage("p2p") as e:
            e["cases"] = p2p_checks(topology, busy_seconds=args.busy_seconds)
            e["ok"] = all(c["ok"] for c in e["cases"])
        with journal.stage("destroy"):
            dist.destroy_process_group()
    except BaseException:
        traceback.print_exc()
        journal.failed = True
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()
    return journal.close()


if __name__ == "__main__":
    sys.exit(main())
