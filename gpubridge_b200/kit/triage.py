"""A short plain-text account of a runbook directory (or a tarball of one), to paste into a review.

    python -m gpubridge_b200.kit.triage results/runbook [--max-lines 80]
    python -m gpubridge_b200.kit.triage results.tgz

Problems first: every step that failed, ran past its limit or was left unfinished, with the
last error lines of its log; then the stage-by-rank verdicts of every check directory whose
summary failed; then what the run was made of (GPUs, torch, NCCL, library) and the numbers
worth a glance - the sweep against NCCL at a few sizes and the weak-scaling table - and one
verdict line.  Host names become ``host N``, IPv4 addresses ``<ip>``; nothing in the input is
executed; needs no torch.  Same purpose as the reference's ``scripts/gpu/triage.py``.
"""
from __future__ import annotations

import argparse
import json
import re
import sys
import tarfile
import tempfile
from pathlib import Path

TAIL = 3
WIDTH = 160
ERROR_LINE = re.compile(r"Error|error:|FAILED|Traceback|timed out|Timeout|refused|mismatch|wrong")


class Redactor:
    def __init__(self) -> None:
        self.hosts: dict[str, str] = {}

    def host(self, name: str) -> str:
        return self.hosts.setdefault(name, f"host {len(self.hosts) + 1}")

    def text(self, line: str) -> str:
        line = re.sub(r"\b\d{1,3}(?:\.\d{1,3}){3}\b", "<ip>", line)
        for name, alias in self.hosts.items():
            if name:
                line = line.replace(name, alias)
        line = re.sub(r"/(home|Users|scratch|work|projects)/[^/\s]+", r"/\1/<owner>", line)
        return line[:WIDTH]


def find_runs(root: Path) -> list[Path]:
    return sorted(p.parent for p in root.rglob("steps.jsonl"))


def last_attempts(path: Path) -> list[dict]:
    rows: dict[str, dict] = {}
    for line in path.read_text().splitlines():
        try:
            row = json.loads(line)
        except json.JSONDecodeError:
            continue
        rows[row["step"]] = row              # a step run again counts as its last attempt
    return list(rows.values())


def error_tail(log: Path, redact: Redactor) -> list[str]:
    if not log.exists():
        return ["(no log)"]
    lines = [l for l in log.read_text(errors="replace").splitlines() if ERROR_LINE.search(l)]
    return [l.strip() for l in lines[-TAIL:]] or ["(no error line in the log)"]


def describe(run: Path, redact: Redactor) -> tuple[list[str], list[str], bool]:
    """(problems, detail, ok) of one runbook directory."""
    problems, detail = [], []
    steps = last_attempts(run / "steps.jsonl")
    probe = run / "probe" / "probe.json"
    env = json.loads(probe.read_text()).get("environment", {}) if probe.exists() else None
    if env:
        redact.host(env.get("hostname", ""))
    logged = {row["log"] for row in steps}
    for row in steps:
        if row["ok"]:
            continue
        what = "ran past its limit" if row["exit_code"] is None else f"exit code {row['exit_code']}"
        problems.append(f"step {row['step']}: FAILED ({what}, {row['seconds']} s)")
        problems += [f"    | {l}" for l in error_tail(run / row["log"], redact)]
    for log in sorted(run.glob("*.log")):
        if log.name not in logged:
            problems.append(f"step {log.stem}: left unfinished (a log without a verdict: the run was killed)")
    for summary in sorted(run.glob("check-*/summary.json")):
        data = json.loads(summary.read_text())
        if not data.get("ok"):
            bad = [f"{stage}: " + ",".join(f"r{r}" for r, ok in ranks.items() if ok is not True)
                   for stage, ranks in data.get("stages", {}).items()
                   if any(ok is not True for ok in ranks.values())]
            problems.append(f"{summary.parent.name}: " + "; ".join(bad[:6]) +
                            (f"; missing ranks {data['ranks_missing']}" if data.get("ranks_missing") else ""))
    if env:
        gpus = sorted({d["name"] for d in env.get("devices", []) if d})
        detail.append(f"ran on {redact.host(env.get('hostname', ''))}: {env.get('device_count')} x "
                      f"{', '.join(gpus) or 'no GPU'}; torch {env.get('torch')}, CUDA {env.get('torch_cuda')}, "
                      f"NCCL {env.get('nccl')}, gpubridge_b200 {env.get('gpubridge_b200')}")
    sweep = run / "sweep.json"
    if sweep.exists():
        rows = json.loads(sweep.read_text())
        by: dict[int, dict[str, dict]] = {}
        for r in rows:
            by.setdefault(int(r["bytes"]), {})[r["target"]] = r
        picked = [b for b in sorted(by) if "ours" in by[b]]
        for b in picked[:: max(1, len(picked) // 4)]:
            ours, nccl = by[b]["ours"], by[b].get("nccl")
            line = f"all_reduce {b} B: ours {ours['ms'] * 1e3:.1f} us ({ours['busbw_gbs']:.1f} GB/s)"
            if nccl:
                line += f", nccl {nccl['ms'] * 1e3:.1f} us, ours = {nccl['ms'] / ours['ms']:.2f}x nccl's speed"
            detail.append(line)
    scaling = run / "scaling" / "summary.json"
    if scaling.exists():
        for row in json.loads(scaling.read_text()).get("rows", []):
            eff = f"{row['efficiency']:.2f}" if row.get("efficiency") is not None else "-"
            detail.append(f"scaling {row['gpus']} GPUs: {row['samples_per_sec']} samples/s, efficiency {eff}, "
                          f"in sync {row['params_in_sync']}")
    gate = run / "gate" / "gate.json"
    if gate.exists():
        g = json.loads(gate.read_text())
        detail.append(f"numerical gate: {'passed' if g['passed'] else 'FAILED ' + '; '.join(g['problems'][:3])}")
        if not g["passed"]:
            problems.append("numerical gate failed: " + "; ".join(g["problems"][:3]))
    return problems, detail, not problems


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("path", type=Path)
    ap.add_argument("--max-lines", type=int, default=80)
    args = ap.parse_args(argv)
    holder = None
    root = args.path
    if root.is_file():
        holder = tempfile.TemporaryDirectory()
        with tarfile.open(root) as tar:
            tar.extractall(holder.name, filter="data")
        root = Path(holder.name)
    redact = Redactor()
    runs = find_runs(root)
    if not runs:
        print(f"no steps.jsonl under {args.path}: not a runbook directory")
        return 2
    problems, detail, verdicts = [], [], []
    for run in runs:
        p, d, ok = describe(run, redact)
        name = run.relative_to(root).as_posix() or "."
        problems += [f"[{name}] {line}" if not line.startswith("    ") else line for line in p]
        detail += [f"[{name}] {line}" for line in d]
        verdicts.append(ok)
    lines = (["PROBLEMS"] + problems if problems else ["no problems found"]) + [""] + detail
    lines += ["", f"verdict: {sum(verdicts)} of {len(verdicts)} run(s) clean"]
    if args.max_lines and len(lines) > args.max_lines:
        keep = args.max_lines - 2
        lines = lines[:keep] + [f"... {len(lines) - keep} more lines (--max-lines 0 for all)", lines[-1]]
    print("\n".join(redact.text(l) for l in lines))      # after every run: all host names are known by now
    if holder is not None:
        holder.cleanup()
    return 0 if all(verdicts) else 1


if __name__ == "__main__":
    sys.exit(main())
