"""The validation runbook for one box: every kit step in order, each under a time limit, one
failure never costing the rest of the session.

    python -m gpubridge_b200.kit.runbook --out results/runbook [--gpus 8] [--dry-run] [--only NAME ...]
    GPUBRIDGE_VENDOR=nvidia python -m gpubridge_b200.kit.runbook --out /tmp/rb --gpus 4 --cpu

Steps (what the reference spreads over ``scripts/gpu/explorer/*.sbatch`` and ``common.sh``):

    probe              environment, library, peer access
    check-<split>      the thirteen-stage check per island split (one island, two halves, and
                       2+2+2+2 / 3+5 on eight GPUs)
    check-<policy>     the same under the pipelined and the sharded policy
    init-error         a negative step: init() must fail with the expected message
    p2p                point-to-point checks through the torch backend, and once more with the
                       C++ front end (GPUBRIDGE_FRONT_END=native)
    gate               the numerical gate (four ranks, both arms)
    streams            the stream-ordering mutation run (one GPU)
    rdma-check         the RDMA-style endpoint's protocol scenarios with injected faults
    sweep              a short all-reduce sweep against NCCL
    scaling            train_synthetic at 1, 2, 4, ... ranks and the weak-scaling table

Every step runs as a child under ``--step-timeout`` seconds (default 1200) with the process
group timeout ``KIT_TIMEOUT`` (default 300) below it, so a stuck collective fails with its
own message first; its output goes to ``<out>/<step>.log`` and its verdict to
``<out>/steps.jsonl``; ``<out>/runbook.md`` is the table.  ``--dry-run`` prints the commands.
Exit code 1 if any step failed.
"""
from __future__ import annotations

import argparse
import json
import os
import re
import subprocess
import sys
import time
from pathlib import Path

PY = sys.executable


def torchrun(n: int, port: int, *rest: str) -> list[str]:
    return [PY, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
            "--master-addr", "127.0.0.1", "--master-port", str(port), *rest]


def plan(out: Path, gpus: int, cpu: bool) -> list[dict]:
    steps: list[dict] = []
    port = [29900]

    def add(name, cmd, env=None, expect=None, timeout=None):
        port[0] += 1
        steps.append({"name": name, "cmd": cmd, "env": env or {}, "expect": expect,
                      "timeout": timeout})
        return port[0]

    add("probe", [PY, "-m", "gpubridge_b200.kit.probe", "--out", str(out / "probe")]
        + (["--allow-no-gpu"] if cpu else []))
    splits = [("one-island", {})]
    if gpus >= 2:
        splits.append(("half", {"GPUBRIDGE_SPLIT_TEST": "half"}))
    if gpus >= 8:
        splits += [("2+2+2+2", {"GPUBRIDGE_ISLANDS": "2,2,2,2"}), ("3+5", {"GPUBRIDGE_ISLANDS": "3,5"})]
    for label, env in splits:
        d = out / f"check-{label}"
        add(f"check-{label}", torchrun(gpus, port[0] + 1, "-m", "gpubridge_b200.kit.check", "--out", str(d))
            + ["--in-flight-settle", "0.5"], env)
        add(f"summary-{label}", [PY, "-m", "gpubridge_b200.kit.summarize", str(d)])
    if gpus >= 2:
        for policy in ("pipelined-reduce-bridge-broadcast", "sharded-bridge"):
            d = out / f"check-{policy}"
            add(f"check-{policy}", torchrun(gpus, port[0] + 1, "-m", "gpubridge_b200.kit.check", "--out",
                                            str(d), "--policy", policy, "--in-flight-settle", "0.5"),
                {"GPUBRIDGE_SPLIT_TEST": "half"})
        add("init-error", torchrun(2, port[0] + 1, "-m", "gpubridge_b200.kit.check", "--out",
                                   str(out / "init-error"), "--expect-init-error",
                                   "problems" if cpu else "apply to this cluster", "--timeout", "60"),
            {"GPUBRIDGE_VENDOR": ""} if cpu else {"GPUBRIDGE_POLICY": "native-only", "GPUBRIDGE_SPLIT_TEST": "half"},
            expect=r"init\(\) failed")
        add("p2p", torchrun(gpus, port[0] + 1, "-m", "gpubridge_b200.kit.check", "--out", str(out / "p2p"),
                            "--p2p-only"), {"GPUBRIDGE_SPLIT_TEST": "half"})
        # the same checks with the C++ c10d::Backend in front of the Python group
        add("p2p-cpp-front-end", torchrun(gpus, port[0] + 1, "-m", "gpubridge_b200.kit.check", "--out",
                                          str(out / "p2p-cpp-front-end"), "--p2p-only"),
            {"GPUBRIDGE_SPLIT_TEST": "half", "GPUBRIDGE_FRONT_END": "native"})
    if gpus >= 4:
        for arm in ("bridged", "native"):
            add(f"gate-{arm}", torchrun(4, port[0] + 1, "-m", "gpubridge_b200.kit.numerical_gate", "--out",
                                        str(out / "gate"), "--arm", arm) + (["--software-only"] if cpu else []))
    if not cpu:
        add("streams", [PY, "-m", "gpubridge_b200.kit.stream_mutations", "--out", str(out / "streams")])
    # the RDMA-style endpoint's protocol scenarios (in-process fabric: needs no adapter and no GPU)
    add("rdma-check", [PY, "-m", "gpubridge_b200.kit.rdma_kit", "check", "--out", str(out / "rdma")])
    if gpus >= 2:
        add("sweep", torchrun(gpus, port[0] + 1, "-m", "gpubridge_b200.bench.bench_all_reduce", "--smallest",
                              "64K", "--largest", "4M" if cpu else "256M", "--trials", "5", "--seconds", "2",
                              "--inner", "4", "--targets", "ours" if cpu else "ours,nccl", "--json",
                              str(out / "sweep.json")))
    n, example = 1, str(Path(__file__).resolve().parents[2] / "examples" / "train_synthetic.py")
    if os.path.exists(example):
        while n <= gpus:
            add(f"scaling-{n}", torchrun(n, port[0] + 1, example, "--json",
                                         str(out / "scaling" / f"train-n{n}.json"), "--steps", "20"))
            n *= 2
        add("scaling-summary", [PY, "-m", "gpubridge_b200.kit.summarize", str(out / "scaling")])
    return steps


def run_step(step: dict, out: Path, limit: float) -> dict:
    env = dict(os.environ, KIT_TIMEOUT=os.environ.get("KIT_TIMEOUT", "300"),
               PYTHONPATH=os.pathsep.join(filter(None, [str(Path(__file__).resolve().parents[2]),
                                                        os.environ.get("PYTHONPATH", "")])))
    for key, value in step["env"].items():
        if value == "":
            env.pop(key, None)
        else:
            env[key] = value
    log = out / f"{step['name']}.log"
    t0 = time.monotonic()
    try:
        done = subprocess.run(step["cmd"], env=env, capture_output=True, text=True,
                              timeout=step["timeout"] or limit)
        text, code = done.stdout + done.stderr, done.returncode
    except subprocess.TimeoutExpired as exc:
        text = f"{exc.stdout or ''}{exc.stderr or ''}\nthe step ran past its limit"
        code = None
    log.write_text(text)
    ok = code == 0 and (step["expect"] is None or re.search(step["expect"], text) is not None)
    return {"step": step["name"], "ok": ok, "exit_code": code,
            "seconds": round(time.monotonic() - t0, 1), "log": log.name}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--out", type=Path, required=True)
    ap.add_argument("--gpus", type=int, default=None)
    ap.add_argument("--cpu", action="store_true", help="CPU ranks (name a vendor with GPUBRIDGE_VENDOR)")
    ap.add_argument("--step-timeout", type=float, default=float(os.environ.get("STEP_TIMEOUT", "1200")))
    ap.add_argument("--only", nargs="*", default=None)
    ap.add_argument("--dry-run", action="store_true")
    args = ap.parse_args(argv)
    gpus = args.gpus
    if gpus is None:
        import torch
        gpus = torch.cuda.device_count() if torch.cuda.is_available() and not args.cpu else 2
    steps = plan(args.out, gpus, args.cpu)
    if args.only:
        steps = [s for s in steps if any(s["name"].startswith(o) for o in args.only)]
    if args.dry_run:
        for s in steps:
            env = " ".join(f"{k}={v}" for k, v in s["env"].items())
            print(f"+ [{s['name']}] {env} {' '.join(s['cmd'])}".replace("  ", " "))
        return 0
    args.out.mkdir(parents=True, exist_ok=True)
    rows = []
    with open(args.out / "steps.jsonl", "a") as journal:
        for s in steps:
            print(f"[runbook] {s['name']} ...", end=" ", flush=True)
            row = run_step(s, args.out, args.step_timeout)
            rows.append(row)
            journal.write(json.dumps(row) + "\n")
            journal.flush()
            print(("ok" if row["ok"] else "FAILED") + f" ({row['seconds']} s)", flush=True)
    lines = ["# Runbook", "", "| step | verdict | seconds | log |", "|---|---|---|---|"]
    lines += [f"| {r['step']} | {'ok' if r['ok'] else 'FAILED'} | {r['seconds']} | {r['log']} |" for r in rows]
    (args.out / "runbook.md").write_text("\n".join(lines) + "\n")
    failed = [r["step"] for r in rows if not r["ok"]]
    print("every step passed" if not failed else f"failed steps: {', '.join(failed)}")
    return 1 if failed else 0


if __name__ == "__main__":
    sys.exit(main())
