"""A small deterministic numerical gate, run under a four-rank torchrun.

    torchrun --nproc-per-node 4 -m gpubridge_b200.kit.numerical_gate --out results/gate
    torchrun --nproc-per-node 4 -m gpubridge_b200.kit.numerical_gate --out results/gate --arm native
    torchrun --nproc-per-node 4 -m gpubridge_b200.kit.numerical_gate --software-only --out results/gate-cpu

Two islands of two ranks (``GPUBRIDGE_SPLIT_TEST=half`` is set here), compression off.
What is checked, per arm (``bridged`` = this package's all-reduce and DDP hook, ``native`` =
``torch.distributed`` on one flat group):

* exact probes: SUM and asynchronous AVG of integer-valued tensors of 17, 65535, 65537 and
  1048577 elements, every element compared (sizes on both sides of the one-shot limit and
  of the pipeline's chunking);
* three steps of a tiny MLP under DDP, with SGD+momentum and with AdamW, against a float64
  replay of the whole batch in one process: gradients, optimizer state and parameters within
  ``1e-6 + 1e-5 * |ref|``, updates within ``2e-8 + 1e-4 * |ref|``;
* three negative controls that must FAIL the same checks (SUM where AVG was asked, a loss
  scaled by two, one rank's inputs shifted), so a gate that cannot fail is noticed.

No performance is measured.  Bounds and probe sizes are those of the reference's
``scripts/gpu/numerical_gate.py`` (:32-37) and ``docs/NUMERICAL_GATE.md``.
"""
from __future__ import annotations

import argparse
import copy
import gc
import hashlib
import json
import os
import socket
import sys
from datetime import datetime, timedelta, timezone
from pathlib import Path

import torch
import torch.distributed as dist
from torch import nn
from torch.nn.parallel import DistributedDataParallel as DDP

import gpubridge_b200 as gb

RTOL, ATOL = 1e-5, 1e-6
UPDATE_RTOL, UPDATE_ATOL = 1e-4, 2e-8
STEPS, BATCH, SEED = 3, 32, 20261020
SIZES = (17, 65535, 65537, 1048577)
ARMS = ("native", "bridged")
CONTROLS = ("none", "sum", "scale", "data")


def fingerprint(named) -> str:
    h = hashlib.sha256()
    for name, t in named:
        t = t.detach().cpu().contiguous()
        h.update(json.dumps([name, list(t.shape), str(t.dtype)]).encode())
        h.update(t.view(torch.uint8).numpy().tobytes())
    return h.hexdigest()


def flat(tensors) -> torch.Tensor:
    return torch.cat([t.detach().cpu().reshape(-1).double() for t in tensors])


def compare(actual, expected, *, exact=False, update=False) -> dict:
    a = torch.as_tensor(actual).detach().cpu().to(torch.float64).reshape(-1)
    b = torch.as_tensor(expected).detach().cpu().to(torch.float64).reshape(-1)
    if a.shape != b.shape:
        return {"violations": max(a.numel(), b.numel()), "shape_mismatch": True}
    delta = (a - b).abs()
    finite = torch.isfinite(a) & torch.isfinite(b)
    atol, rtol = (UPDATE_ATOL, UPDATE_RTOL) if update else (ATOL, RTOL)
    bad = (~finite) | (delta > (0 if exact else atol + rtol * b.abs()))
    clean = bool(finite.all())
    return {"violations": int(bad.sum()), "elements": a.numel(),
            "max_abs": float(delta.max()) if clean else None,
            "relative_l2": float(torch.linalg.vector_norm(a - b)
                                 / torch.linalg.vector_norm(b).clamp_min(1e-30)) if clean else None}


def tiny_model() -> nn.Module:
    torch.manual_seed(SEED)
    m = nn.Sequential(nn.Linear(6, 5, bias=False), nn.Tanh(), nn.Linear(5, 3, bias=False))
    with torch.no_grad():
        for p in m.parameters():
            p.copy_(torch.randint(-3, 4, p.shape).float() / 16)
    return m


def global_batch(step: int):
    g = torch.Generator().manual_seed(SEED + 100 + step)
    return (torch.randint(-8, 9, (BATCH, 6), generator=g).float() / 8,
            torch.randint(-8, 9, (BATCH, 3), generator=g).float() / 8)


def make_optimizer(params, name: str):
    if name == "sgd":
        return torch.optim.SGD(params, lr=1 / 32, momentum=0.5, foreach=False)
    return torch.optim.AdamW(params, lr=1e-3, weight_decay=0.01, eps=1e-8, foreach=False,
                             fused=False)


def optimizer_state(opt) -> list[torch.Tensor]:
    return [state[k] for group in opt.param_groups for p in group["params"]
            for state in [opt.state[p]] for k in sorted(state)
            if isinstance(state[k], torch.Tensor)]


def run_gate(topology, *, arm: str, software_only: bool, opt_name: str = "sgd",
             control: str = "none", sizes=SIZES) -> dict:
    """Every rank calls this; a numerical violation is recorded, never raised."""
    rank, world = dist.get_rank(), dist.get_world_size()
    if world != 4:
        raise ValueError("the gate is defined for four ranks")
    device = topology.device if topology is not None else torch.device(
        "cpu" if software_only else f"cuda:{int(os.environ.get('LOCAL_RANK', 0))}")
    if device.type == "cuda":
        torch.cuda.set_device(device)
    torch.set_num_threads(1)
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    report = {"schema": "gpubridge_b200.numerical_gate/1", "arm": arm, "rank": rank,
              "world": world, "software_only": software_only, "control": control,
              "optimizer": opt_name, "seed": SEED, "steps": STEPS, "global_batch": BATCH,
              "probe_sizes": list(sizes), "rtol": RTOL, "atol": ATOL, "update_rtol": UPDATE_RTOL,
              "update_atol": UPDATE_ATOL, "device": str(device), "host": socket.gethostname(),
              "torch": torch.__version__,
              "gpu": torch.cuda.get_device_name(device) if device.type == "cuda" else None,
              "checks": [], "errors": [], "inputs": [],
              "created_at": datetime.now(timezone.utc).isoformat()}
    if topology is not None:
        layout = [list(i.ranks) for i in topology.layout.islands]
        report.update(layout=layout, policy=topology.policy_name, run_kind=topology.run_kind,
                      fused=topology.fabric is not None,
                      transport=topology.peers[rank].bridge)
        if layout != [[0, 1], [2, 3]] or topology.bridge_compression:
            raise ValueError("the bridged arm needs two islands of two and compression off")
    else:
        report.update(layout=[[0, 1, 2, 3]], policy="native", run_kind="native", fused=False,
                      transport="native")

    def check(label, actual, expected, exact=False):
        report["checks"].append({"name": label, **compare(actual, expected, exact=exact,
                                                           update=label.startswith("update/"))})

    # exact probes; the AVG calls are queued together and waited for afterwards
    pending = []
    for n in sizes:
        base = torch.arange(n, dtype=torch.float32)
        want = world * base + world * (world + 1) / 2
        for average in (False, True):
            t = (base + rank + 1).to(device)
            if topology is None:
                work = dist.all_reduce(t, async_op=average)
            else:
                work = gb.all_reduce(t, op=gb.ReduceOp.AVG if average else gb.ReduceOp.SUM,
                                     async_op=average)
            if average:
                pending.append((n, t, want / world, work))
            else:
                check(f"sum/{n}", t, want, exact=True)
    for n, t, want, work in pending:
        work.wait()
        if topology is None:
            t.div_(world)
        if control == "sum":
            t.mul_(world)
        check(f"avg/{n}", t, want, exact=True)

    first = tiny_model()
    first_hash = fingerprint(first.named_parameters())
    oracle = copy.deepcopy(first).double()
    model = first.to(device)
    ddp = DDP(model, device_ids=[device.index] if device.type == "cuda" else None,
              broadcast_buffers=False, bucket_cap_mb=0.00005)
    if topology is not None:
        ddp.register_comm_hook(None, gb.ddp_comm_hook)
    report["initial_sha256"] = first_hash
    if fingerprint(model.named_parameters()) != first_hash:
        report["errors"].append("DDP changed the initial parameters")
    opt, oracle_opt = make_optimizer(ddp.parameters(), opt_name), make_optimizer(
        oracle.parameters(), opt_name)
    share = BATCH // world
    for step in range(STEPS):
        x, y = global_batch(step)
        rows = slice(rank * share, (rank + 1) * share)
        lx, ly = x[rows].clone(), y[rows].clone()
        want_hash = fingerprint([("x", lx), ("y", ly)])
        if control == "data" and rank == 0:
            lx.add_(1 / 8)
        got_hash = fingerprint([("x", lx), ("y", ly)])
        report["inputs"].append({"step": step, "expected": want_hash, "actual": got_hash})
        if got_hash != want_hash:
            report["errors"].append(f"input fingerprint mismatch at step {step}")
        opt.zero_grad(set_to_none=True)
        oracle_opt.zero_grad(set_to_none=True)
        loss = (ddp(lx.to(device)) * ly.to(device)).sum(1).mean()
        (loss * (2 if control == "scale" else 1)).backward()
        (oracle(x.double()) * y.double()).sum(1).mean().backward()
        params, twins = list(model.parameters()), list(oracle.parameters())
        check(f"gradient/{step}", flat(p.grad for p in params), flat(p.grad for p in twins))
        old, old_twin = [p.detach().clone() for p in params], [p.detach().clone() for p in twins]
        opt.step()
        oracle_opt.step()
        check(f"update/{step}", flat(p - q for p, q in zip(params, old, strict=True)),
              flat(p - q for p, q in zip(twins, old_twin, strict=True)))
        check(f"parameters/{step}", flat(params), flat(twins))
        check(f"optimizer_state/{step}", flat(optimizer_state(opt)),
              flat(optimizer_state(oracle_opt)))
    report["final_sha256"] = fingerprint(model.named_parameters())
    report["passed"] = not report["errors"] and not any(c["violations"] for c in report["checks"])
    del ddp, model, opt
    gc.collect()
    return report


def verdict(records: list[dict]) -> dict:
    """Merge the ranks' records of one invocation: positive runs must pass on every rank and
    agree on the final parameters; every negative control must fail somewhere."""
    problems = []
    groups: dict[tuple, list[dict]] = {}
    for r in records:
        groups.setdefault((r["arm"], r["optimizer"], r["control"]), []).append(r)
    for (arm, opt, control), rows in sorted(groups.items()):
        if len(rows) != 4:
            problems.append(f"{arm}/{opt}/{control}: {len(rows)} of 4 rank records")
        if control == "none":
            for r in rows:
                if not r["passed"]:
                    bad = [c["name"] for c in r["checks"] if c["violations"]] + r["errors"]
                    problems.append(f"{arm}/{opt} rank {r['rank']}: {bad[:6]}")
            if len({r["final_sha256"] for r in rows}) != 1:
                problems.append(f"{arm}/{opt}: ranks disagree on the final parameters")
        elif all(r["passed"] for r in rows):
            problems.append(f"{arm}/{opt}: negative control {control!r} passed; the gate cannot "
                            "see that fault")
    return {"passed": not problems, "problems": problems, "runs": sorted(
        f"{a}/{o}/{c}" for a, o, c in groups)}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--out", type=Path, required=True)
    ap.add_argument("--software-only", action="store_true", help="CPU ranks over Gloo")
    ap.add_argument("--arm", default="bridged", choices=ARMS,
                    help="one arm per invocation; run again with the other arm into the same "
                         "--out and the verdict covers both")
    ap.add_argument("--timeout", type=float, default=300)
    args = ap.parse_args(argv)
    os.environ.setdefault("GPUBRIDGE_SPLIT_TEST", "half")
    if args.software_only:
        os.environ.setdefault("GPUBRIDGE_VENDOR", "nvidia")
    rank = int(os.environ.get("RANK", "0"))
    records = []
    if args.arm == "native":
        dist.init_process_group("gloo" if args.software_only else "nccl",
                                timeout=timedelta(seconds=args.timeout))
        topology = None
    else:
        topology = gb.init(timeout=timedelta(seconds=args.timeout))
    try:
        for opt_name in ("sgd", "adamw"):
            records.append(run_gate(topology, arm=args.arm, software_only=args.software_only,
                                    opt_name=opt_name))
        for control in CONTROLS[1:]:
            records.append(run_gate(topology, arm=args.arm, software_only=args.software_only,
                                    opt_name="sgd", control=control, sizes=SIZES[:2]))
        args.out.mkdir(parents=True, exist_ok=True)
        mine = args.out / f"gate-{args.arm}-rank{rank}.json"
        tmp = mine.with_suffix(".tmp")
        tmp.write_text(json.dumps(records, indent=1))
        tmp.replace(mine)
        dist.barrier() if topology is None else gb.barrier()
    finally:
        if topology is None:
            dist.destroy_process_group()
        else:
            gb.destroy()
    if rank != 0:
        return 0
    merged = []
    for path in sorted(args.out.glob("gate-*-rank*.json")):
        merged += json.loads(path.read_text())
    result = verdict(merged)
    (args.out / "gate.json").write_text(json.dumps(result, indent=1))
    print(json.dumps(result))
    return 0 if result["passed"] else 1


if __name__ == "__main__":
    sys.exit(main())
