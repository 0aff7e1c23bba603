"""The hardware-validation tables, from what the kit's jobs left behind.

    python -m gpubridge_b200.kit.validation_tables results/slurm [more paths ...] [--out DIR]

Every directory under the paths that holds a ``steps.jsonl`` (a ``kit.runbook`` directory or a
Slurm job's) is one job.  Writes ``validation_tables.md`` and ``validation_tables.json`` into
``--out`` (default: the first path):

* **Runs** - per job: steps passed / failed, and what it ran on (hosts, numbered in order of
  appearance; GPU models; torch, CUDA, NCCL, this library's version).
* **Items** - the validation items (below), each with the steps and check stages that test it
  and how they went across every job: *passed* (on GPUs), *FAILED*, *simulation only* or
  *not run*.  A CPU-simulation result never counts towards an item: it says nothing about GPUs.
* **Network** - the preflight's chosen interface, round trip and bandwidth each way.
* **Benchmarks** - the fused all-reduce against NCCL at a few sizes.
* **Predicted vs measured** - for bridged jobs with a preflight: the time the preflight's
  bandwidth predicts for moving each size across the bridge once each way, beside the
  all-reduce the sweep measured (a bridge that is much slower than its link shows here).

Hosts are numbered and no path is shown: the tables can be published; the raw records keep
the names.  Same purpose as the reference's ``scripts/gpu/validation_tables.py``.
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

#: item -> (what it establishes, steps whose verdict counts, check stages whose verdict counts)
ITEMS = [
    ("build", "the native library builds for sm_100a, loads, and matches its bindings", ("probe",), ()),
    ("placement", "one process per GPU lands on the GPU it was given", ("probe",), ("device",)),
    ("discovery", "ranks find their islands, leaders and the bridge", (), ("init",)),
    ("dtypes", "every supported dtype reduces exactly", (), ("dtypes",)),
    ("stream-order", "collectives are ordered with the caller's stream (busy GPU, poisoned buffers)",
     ("streams",), ("busy_gpu",)),
    ("collectives", "broadcast, reductions, all_gather, reduce_scatter give the exact answer",
     (), ("broadcast", "reductions", "all_gather", "reduce_scatter")),
    ("async", "async work handles, in-flight accounting, bit-identical results on every rank",
     (), ("async", "in_flight", "reduction_agreement")),
    ("teardown", "barrier and destroy leave nothing behind", (), ("barrier", "destroy")),
    ("policies", "pipelined and sharded bridge policies agree with the default",
     ("check-pipelined-reduce-bridge-broadcast", "check-sharded-bridge"), ()),
    ("negative-init", "a configuration that cannot work fails on every rank with its reason", ("init-error",), ()),
    ("p2p", "send / recv / batched P2P through the torch backend", ("p2p",), ()),
    ("cpp-front-end", "the same through the C++ c10d::Backend", ("p2p-cpp-front-end",), ()),
    ("numerics", "training numerics inside the gate's bounds, controls fail as they must",
     ("gate-bridged", "gate-native"), ()),
    ("performance", "all-reduce sweep against NCCL", ("sweep",), ()),
    ("scaling", "data-parallel replicas stay bit-identical; weak scaling", ("scaling-summary",), ()),
    ("cross-node", "two boxes joined by a host bridge (preflight, Gloo and multi-stream TCP bridges)",
     ("preflight", "check-gloo", "check-multitcp"), ()),
]
SIZES = (1 << 16, 1 << 20, 1 << 24, 1 << 28)


class Hosts:
    def __init__(self) -> None:
        self.seen: dict[str, str] = {}

    def __call__(self, name: str) -> str:
        return self.seen.setdefault(name or "?", f"host {len(self.seen) + 1}")


def read(path: Path):
    try:
        return json.loads(path.read_text())
    except (OSError, json.JSONDecodeError):
        return None


def load_job(directory: Path, hosts: Hosts) -> dict:
    steps: dict[str, dict] = {}
    for line in (directory / "steps.jsonl").read_text().splitlines():
        try:
            row = json.loads(line)
            steps[row["step"]] = row
        except (json.JSONDecodeError, KeyError):
            continue
    stages: dict[str, list[bool]] = {}          # check stage -> verdicts over every check directory
    simulated, environments = None, []
    for summary in sorted(directory.glob("*/summary.json")):
        data = read(summary) or {}
        if "stages" not in data:
            continue
        for stage, ranks in data["stages"].items():
            stages.setdefault(stage, []).append(all(v is True for v in ranks.values())
                                                and not data.get("ranks_missing"))
    for record in sorted(directory.glob("*/rank0.json")) + sorted(directory.glob("probe/probe.json")):
        env = (read(record) or {}).get("environment")
        if env:
            environments.append(env)
    env = environments[0] if environments else {}
    # a job counts as a GPU job only when its ranks ran on GPUs: a record says so itself
    simulated = not (environments and all(e.get("cuda_available") and e.get("device_count") for e in environments))
    if any("GPUBRIDGE_VENDOR" in (e.get("env") or {}) for e in environments):
        simulated = True
    gpus = sorted({d["name"] for e in environments for d in e.get("devices", []) if d})
    return {"steps": steps, "stages": stages, "simulated": bool(simulated),
            "hosts": sorted({hosts(e.get("hostname", "")) for e in environments}),
            "gpus": gpus, "gpu_count": env.get("device_count"),
            "software": {k: env.get(k) for k in ("torch", "torch_cuda", "nccl", "gpubridge_b200")},
            "preflight": read(directory / "preflight" / "preflight-master.json"),
            "sweep": read(directory / "sweep.json")}


def item_state(job: dict, steps, stages) -> str | None:
    """passed / FAILED / None (nothing of this item ran in this job)."""
    verdicts = [job["steps"][s]["ok"] for s in steps if s in job["steps"]]
    verdicts += [ok for s in stages for ok in job["stages"].get(s, [])]
    if not verdicts:
        return None
    return "passed" if all(verdicts) else "FAILED"


def tables(jobs: dict[str, dict]) -> tuple[dict, str]:
    out: dict = {"runs": [], "items": [], "network": [], "benchmarks": [], "predicted_vs_measured": []}
    md = ["# Hardware validation", ""]
    md += ["## Runs", "", "| job | kind | steps passed | steps failed | ran on | GPUs | software |", "|---|---|---|---|---|---|---|"]
    for name, job in jobs.items():
        good = [s for s, r in job["steps"].items() if r["ok"]]
        bad = [s for s, r in job["steps"].items() if not r["ok"]]
        soft = job["software"]
        row = {"job": name, "simulation": job["simulated"], "passed": good, "failed": bad, "hosts": job["hosts"],
               "gpus": job["gpus"], "gpu_count": job["gpu_count"], "software": soft}
        out["runs"].append(row)
        md.append(f"| {name} | {'CPU simulation' if job['simulated'] else 'GPU'} | {len(good)} | "
                  f"{', '.join(bad) or '-'} | {', '.join(job['hosts']) or '-'} | "
                  f"{job['gpu_count'] or 0} x {', '.join(job['gpus']) or '-'} | "
                  + (f"torch {soft['torch']}, CUDA {soft['torch_cuda']}, NCCL {soft['nccl']}, "
                     f"gpubridge_b200 {soft['gpubridge_b200']}" if soft["torch"] else "- (see its steps' own rows)")
                  + " |")
    md += ["", "## Items", "", "| item | establishes | verdict | where |", "|---|---|---|---|"]
    for key, meaning, steps, stages in ITEMS:
        where, gpu_states, sim_states = [], [], []
        for name, job in jobs.items():
            state = item_state(job, steps, stages)
            if state is None:
                continue
            (sim_states if job["simulated"] else gpu_states).append(state)
            where.append(f"{name}: {state}{' (simulation)' if job['simulated'] else ''}")
        if "FAILED" in gpu_states + sim_states:
            verdict = "FAILED"
        elif gpu_states:
            verdict = "passed"
        elif sim_states:
            verdict = "simulation only"
        else:
            verdict = "not run"
        out["items"].append({"item": key, "verdict": verdict, "where": where})
        md.append(f"| {key} | {meaning} | {verdict} | {'; '.join(where) or '-'} |")
    flights = [(n, j["preflight"]) for n, j in jobs.items() if j["preflight"]]
    if flights:
        md += ["", "## Network", "", "| job | interface | round trip, us | out, MB/s | in, MB/s | Gloo pair |", "|---|---|---|---|---|---|"]
        for name, p in flights:
            band = p.get("bandwidth") or {}
            row = {"job": name, "ifname": p.get("chosen_ifname"), "rtt_us": band.get("rtt_us"),
                   "out_MBps": band.get("out_MBps"), "in_MBps": band.get("in_MBps"),
                   "gloo": p.get("checks", {}).get("gloo")}
            out["network"].append(row)
            md.append(f"| {name} | {row['ifname']} | {row['rtt_us']} | {row['out_MBps']} | {row['in_MBps']} | {row['gloo']} |")
    sweeps = [(n, j) for n, j in jobs.items() if j["sweep"]]
    if sweeps:
        md += ["", "## Benchmarks", "", "| job | bytes | ours, us | ours busbw, GB/s | NCCL, us | ours / NCCL speed |", "|---|---|---|---|---|---|"]
        for name, job in sweeps:
            by: dict[int, dict] = {}
            for r in job["sweep"]:
                by.setdefault(int(r["bytes"]), {})[r["target"]] = r
            have = sorted(b for b in by if "ours" in by[b])
            for want in SIZES:
                near = min(have, key=lambda b: abs(b - want), default=None)
                if near is None or not want / 2 <= near <= want * 2:
                    continue
                ours, nccl = by[near]["ours"], by[near].get("nccl")
                row = {"job": name, "simulation": job["simulated"], "bytes": near, "ours_us": round(ours["ms"] * 1e3, 1),
                       "ours_busbw_gbs": ours.get("busbw_gbs"), "nccl_us": round(nccl["ms"] * 1e3, 1) if nccl else None,
                       "speed_vs_nccl": round(nccl["ms"] / ours["ms"], 2) if nccl else None}
                out["benchmarks"].append(row)
                md.append(f"| {name}{' (simulation)' if job['simulated'] else ''} | {near} | {row['ours_us']} | "
                          f"{row['ours_busbw_gbs']} | {row['nccl_us'] or '-'} | {row['speed_vs_nccl'] or '-'} |")
                flight = job["preflight"]
                band = (flight or {}).get("bandwidth") or {}
                slow = min((v for v in (band.get("out_MBps"), band.get("in_MBps")) if v), default=None)
                if slow:
                    predicted = near / (slow * 1e6) * 1e6 + (band.get("rtt_us") or 0.0)
                    out["predicted_vs_measured"].append(
                        {"job": name, "bytes": near, "bridge_predicted_us": round(predicted, 1),
                         "all_reduce_measured_us": row["ours_us"], "ratio": round(row["ours_us"] / predicted, 2)})
    if out["predicted_vs_measured"]:
        md += ["", "## Predicted vs measured", "",
               "Predicted: one crossing of the bridge at the preflight's slower direction plus one round trip "
               "(one TCP stream driven from Python: a lower bound on the link).  Measured: the whole all-reduce.",
               "", "| job | bytes | bridge predicted, us | all-reduce measured, us | measured / predicted |", "|---|---|---|---|---|"]
        md += [f"| {r['job']} | {r['bytes']} | {r['bridge_predicted_us']} | {r['all_reduce_measured_us']} | {r['ratio']} |"
               for r in out["predicted_vs_measured"]]
    return out, "\n".join(md) + "\n"


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("paths", nargs="+", type=Path)
    ap.add_argument("--out", type=Path)
    args = ap.parse_args(argv)
    hosts = Hosts()
    jobs: dict[str, dict] = {}
    for root in args.paths:
        for journal in sorted(root.rglob("steps.jsonl")):
            name = journal.parent.relative_to(root).as_posix()
            jobs[name if name != "." else root.name] = load_job(journal.parent, hosts)
    if not jobs:
        print("no steps.jsonl under the given paths")
        return 2
    data, text = tables(jobs)
    out = args.out or args.paths[0]
    out.mkdir(parents=True, exist_ok=True)
    (out / "validation_tables.md").write_text(text)
    (out / "validation_tables.json").write_text(json.dumps(data, indent=1))
    print(text, end="")
    return 1 if any(i["verdict"] == "FAILED" for i in data["items"]) else 0


if __name__ == "__main__":
    sys.exit(main())
