"""Merge the per-rank journals of a kit run into ``summary.json`` and ``summary.md``.

    python -m gpubridge_b200.kit.summarize [--partial] DIR [DIR ...]

A directory of ``rank<N>.json`` journals gets a stage-by-rank table; exit code 1 if a rank is
missing, a stage failed or a rank was left inside a stage.  Relabelled (split-test) runs are
flagged at the top.  ``--partial``: this machine holds only some ranks of a multi-machine
job; absent ranks are listed, not failed.  Same role as the reference's
``scripts/gpu/summarize.py``.
"""
from __future__ import annotations

import json
import re
import sys
from pathlib import Path
from typing import Any

from gpubridge_b200.kit import write_json

BANNER = ("> **SPLIT TEST - not a mixed-vendor result.** The islands are relabelled ranks of "
          "a single-vendor job.")
_MARK = {True: "ok", False: "FAIL", None: "-"}


def load(directory: Path) -> dict[int, dict[str, Any]]:
    journals = {}
    for path in directory.glob("rank*.json"):
        m = re.fullmatch(r"rank(\d+)\.json", path.name)
        if m:
            journals[int(m.group(1))] = json.loads(path.read_text())
    return journals


def summarize(directory: Path, partial: bool = False) -> tuple[dict[str, Any], str]:
    journals = load(directory)
    runs = [j["run"] for j in journals.values() if j.get("run")]
    world = runs[0]["world_size"] if runs else None
    missing = sorted(set(range(world)) - set(journals)) if world else []
    split = next((r["split_test"] for r in runs if r.get("split_test")), None)
    stage_names: list[str] = []
    for j in journals.values():
        for s in j["stages"]:
            if s["name"] not in stage_names:
                stage_names.append(s["name"])
    problems: dict[str, str] = {}
    for rank, j in sorted(journals.items()):
        for s in j["stages"]:
            where = f"rank {rank} / {s['name']}"
            if s["ok"] is False:
                problems[where] = s.get("error") or json.dumps(
                    {k: v for k, v in s.items() if k not in ("name", "ok")}, default=str)
            elif s["ok"] is None:
                problems[where] = "the rank was left inside this stage"
    if not split:
        # two ranks on one physical GPU is a mistake of the launch unless the run relabels on purpose
        holders: dict[tuple, list[int]] = {}
        for rank, j in sorted(journals.items()):
            device = (j.get("run") or {}).get("device") or ""
            if not device.startswith("cuda"):
                continue
            index = int(device.split(":")[1]) if ":" in device else 0
            devices = (j.get("environment") or {}).get("devices") or []
            bus = next((d.get("pci_bus_id") for d in devices if d and d.get("index") == index), None)
            if bus:
                holders.setdefault(((j.get("environment") or {}).get("hostname"), bus), []).append(rank)
        for (host, bus), ranks in holders.items():
            if len(ranks) > 1:
                problems[f"ranks {ranks}"] = (f"share one GPU (PCI {bus} on {host}) outside a split test: "
                                              "give every rank its own device")
    table = {name: {rank: next((s["ok"] for s in j["stages"] if s["name"] == name), None)
                    for rank, j in sorted(journals.items())} for name in stage_names}
    ok = (bool(journals) and (partial or not missing) and not problems
          and all(j.get("ok") for j in journals.values()))
    first = journals[min(journals)] if journals else {}
    summary = {
        "directory": str(directory), "ok": ok, "run_kind": runs[0]["kind"] if runs else "unknown",
        "policy": runs[0].get("policy") if runs else None, "split_test": split,
        "fused": runs[0].get("fused") if runs else None,
        "ranks_reported": sorted(journals), "ranks_missing": missing, "partial": partial,
        "islands": runs[0]["islands"] if runs else None,
        "environment": {k: first.get("environment", {}).get(k)
                        for k in ("torch", "torch_cuda", "nccl", "gpubridge_b200")},
        "stages": table, "errors": problems,
    }
    lines = [f"# {directory.name}: {'PASS' if ok else 'FAIL'}", ""]
    if split:
        lines += [BANNER, ""]
    lines += [f"Run kind `{summary['run_kind']}`, policy `{summary['policy']}`, fused kernels "
              f"`{summary['fused']}`, split test `{split or 'off'}`, "
              f"{len(journals)}{f' of {world}' if world else ''} ranks reported.", ""]
    if missing:
        lines += [(f"Ranks {missing} ran on another machine (partial summary)." if partial else
                   f"**Missing ranks:** {missing} (died before writing a journal?)"), ""]
    lines += ["| stage | " + " | ".join(f"rank {r}" for r in sorted(journals)) + " |",
              "|" + " --- |" * (len(journals) + 1)]
    for name, row in table.items():
        lines.append(f"| {name} | " + " | ".join(_MARK[v] for v in row.values()) + " |")
    if problems:
        lines += ["", "## Problems", ""]
        for where, what in problems.items():
            lines += [f"* **{where}**", "", "```", what.strip()[-2000:], "```", ""]
    return summary, "\n".join(lines) + "\n"


def summarize_scaling(directory: Path) -> tuple[dict[str, Any], str]:
    """Weak-scaling table from ``train-n<N>.json`` records (examples/train_synthetic.py)."""
    runs = {}
    for path in directory.glob("train-n*.json"):
        record = json.loads(path.read_text())
        runs[record["world_size"]] = record
    base = runs.get(1, {}).get("samples_per_sec")
    rows = []
    for n, record in sorted(runs.items()):
        rate = record.get("samples_per_sec")
        rows.append({"gpus": n, "samples_per_sec": rate,
                     "efficiency": rate / (n * base) if base and rate else None,
                     "step_ms_median": record.get("step_ms_median"),
                     "params_in_sync": record.get("params_in_sync"),
                     "split_test": (record.get("run") or {}).get("split_test")})
    split = next((r["split_test"] for r in rows if r["split_test"]), None)
    ok = bool(rows) and all(r["params_in_sync"] for r in rows)
    lines = [f"# {directory.name}: scaling", ""]
    if split:
        lines += [BANNER, ""]
    lines += ["Weak scaling: fixed batch per GPU; efficiency = samples/s on N GPUs / (N x samples/s "
              "on 1 GPU).", "", "| GPUs | samples/s | efficiency | median step (ms) | parameters in sync |",
              "| --- | --- | --- | --- | --- |"]
    for r in rows:
        eff = f"{r['efficiency']:.2f}" if r["efficiency"] is not None else "-"
        lines.append(f"| {r['gpus']} | {r['samples_per_sec']} | {eff} | {r['step_ms_median']} | "
                     f"{r['params_in_sync']} |")
    return {"directory": str(directory), "ok": ok, "split_test": split, "rows": rows}, "\n".join(lines) + "\n"


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    partial = "--partial" in argv
    if "-h" in argv or "--help" in argv:
        print(__doc__)
        return 0
    dirs = [Path(a) for a in argv if a != "--partial"]
    if not dirs or any(str(d).startswith("-") for d in dirs):
        print(__doc__, file=sys.stderr)
        return 2
    failed = False
    for d in dirs:
        if any(d.glob("train-n*.json")):
            summary, text = summarize_scaling(d)
        else:
            summary, text = summarize(d, partial)
        write_json(d / "summary.json", summary)
        (d / "summary.md").write_text(text)
        print(text)
        failed = failed or not summary["ok"]
    return 1 if failed else 0


if __name__ == "__main__":
    sys.exit(main())
