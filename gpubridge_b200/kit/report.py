"""Tables over training records: runs side by side against a baseline, and replica-divergence
verdicts.  Needs only the standard library.

    python -m gpubridge_b200.kit.report dp  DIR [DIR ...] --out OUT [--baseline FILE]
    python -m gpubridge_b200.kit.report ddp DIR [DIR ...] [--out OUT]

``dp``: every JSON record under the paths written by ``bench.train_dp --json`` or
``bench.train_pipeline --json`` is a run; the one with ``"mode": "single"`` is the baseline.
Per run: mode, compression, shares, tokens/s from the median step, speed-up over the
baseline, the last loss, the largest gap to the baseline's loss curve over every step and the
mean gap over the last steps, and whether every parameter check found the replicas identical.
Writes ``dp_report.md``, ``loss_curves.csv`` and ``loss_curves.svg``.  (The reference's
``scripts/gpu/dp_report.py``.)

``ddp``: every record written by ``examples/train_synthetic.py --json`` is a run.  Per run a
verdict from the bit-for-bit checks it made after every step: *in sync*; *gradients differ
after all_reduce* (the synced gradients already differed: look at the exchange - bridge,
compression); *parameters differ, gradients equal* (the optimizer turned the same gradients
into different parameters); *no per-step check* for records without them.  Exit code 1 when
any run diverged.  (The reference's ``scripts/gpu/train_ddp_report.py``.)
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

PALETTE = ("#3366cc", "#dc3912", "#109618", "#990099", "#ff9900", "#0099c6", "#dd4477", "#66aa00")


def records(paths, accept) -> list[tuple[str, dict]]:
    found = []
    for root in paths:
        files = [root] if root.is_file() else sorted(root.rglob("*.json"))
        for f in files:
            try:
                data = json.loads(f.read_text())
            except (OSError, json.JSONDecodeError):
                continue
            if isinstance(data, dict) and accept(data):
                found.append((f.stem if root.is_file() else f.relative_to(root).with_suffix("").as_posix(), data))
    return found


# -- dp ---------------------------------------------------------------------------------------------
def label(name: str, r: dict) -> str:
    if r.get("bench") == "train_pipeline":
        return f"{name}: pipeline {r.get('schedule')} x{r.get('stages')}"
    bits = [r.get("mode", "?"), f"x{r.get('world', 1)}"]
    if r.get("compression"):
        bits.append(r["compression"])
    return f"{name}: " + " ".join(bits)


def curve_gaps(losses: list[float], base: list[float], tail: int) -> tuple[float, float]:
    n = min(len(losses), len(base))
    gaps = [abs(a - b) for a, b in zip(losses[:n], base[:n])]
    last = gaps[-min(tail, n):]
    return max(gaps), sum(last) / len(last)


def svg(curves: list[tuple[str, list[float]]], width=760, height=420) -> str:
    left, top, right, bottom = 56, 16, 200, 36
    steps = max(len(c) for _, c in curves)
    lo = min(min(c) for _, c in curves)
    hi = max(max(c) for _, c in curves)
    span = (hi - lo) or 1.0
    w, h = width - left - right, height - top - bottom

    def at(i, v):
        return left + w * i / max(1, steps - 1), top + h * (1 - (v - lo) / span)

    out = [f'<svg xmlns="http://www.w3.org/2000/svg" width="{width}" height="{height}" font-family="sans-serif" font-size="11">',
           f'<rect width="{width}" height="{height}" fill="white"/>',
           f'<path d="M{left},{top}V{top + h}H{left + w}" fill="none" stroke="#444"/>']
    for k in range(5):
        v = lo + span * k / 4
        y = at(0, v)[1]
        out.append(f'<text x="{left - 6}" y="{y + 4:.1f}" text-anchor="end">{v:.3f}</text>')
        out.append(f'<path d="M{left},{y:.1f}H{left + w}" stroke="#ddd"/>')
    out.append(f'<text x="{left + w / 2}" y="{height - 8}" text-anchor="middle">step</text>')
    for n, (name, c) in enumerate(curves):
        colour = PALETTE[n % len(PALETTE)]
        points = " ".join(f"{x:.1f},{y:.1f}" for x, y in (at(i, v) for i, v in enumerate(c)))
        out.append(f'<polyline points="{points}" fill="none" stroke="{colour}" stroke-width="1.4"/>')
        out.append(f'<text x="{left + w + 10}" y="{top + 14 + 15 * n}" fill="{colour}">{name[:30]}</text>')
    return "\n".join(out + ["</svg>"]) + "\n"


def dp_report(paths, out: Path, baseline: Path | None, tail: int) -> int:
    runs = records(paths, lambda d: d.get("bench") in ("train_dp", "train_pipeline") and "losses" in d)
    if not runs:
        print("no recorded train_dp / train_pipeline runs found")
        return 2
    if baseline is not None:
        base = json.loads(baseline.read_text())
    else:
        singles = [r for _, r in runs if r.get("mode") == "single"]
        base = singles[0] if singles else None
    lines = ["# Training runs side by side", ""]
    if base is None:
        lines += ["No single-GPU baseline among the records: speed-ups and loss gaps are left out.", ""]
    lines += ["| run | global batch | shares | tokens/s | vs baseline | last loss | largest loss gap | "
              f"mean gap, last {tail} | replicas identical |", "|---|---|---|---|---|---|---|---|---|"]
    for name, r in runs:
        speed = gap = mean = "-"
        if base is not None and r is not base:
            speed = f"{r['tokens_per_s'] / base['tokens_per_s']:.2f}x"
            worst, late = curve_gaps(r["losses"], base["losses"], tail)
            gap, mean = f"{worst:.2e}", f"{late:.2e}"
        same = r.get("parameters_identical")
        lines.append(f"| {label(name, r)}{' (baseline)' if r is base else ''} | {r.get('global_batch')} | "
                     f"{r.get('shares') or r.get('split') or '-'} | {r['tokens_per_s']} | {speed} | "
                     f"{r['losses'][-1]:.4f} | {gap} | {mean} | "
                     f"{'-' if same is None else 'yes' if same else 'NO'} |")
    out.mkdir(parents=True, exist_ok=True)
    (out / "dp_report.md").write_text("\n".join(lines) + "\n")
    steps = max(len(r["losses"]) for _, r in runs)
    rows = ["step," + ",".join(label(n, r).replace(",", ";") for n, r in runs)]
    for i in range(steps):
        rows.append(f"{i}," + ",".join(f"{r['losses'][i]:.6f}" if i < len(r["losses"]) else "" for _, r in runs))
    (out / "loss_curves.csv").write_text("\n".join(rows) + "\n")
    (out / "loss_curves.svg").write_text(svg([(label(n, r), r["losses"]) for n, r in runs]))
    print("\n".join(lines))
    diverged = [n for n, r in runs if r.get("parameters_identical") is False]
    return 1 if diverged else 0


# -- ddp --------------------------------------------------------------------------------------------
def ddp_verdict(r: dict) -> str:
    if "first_gradient_difference" not in r and "first_parameter_difference" not in r:
        return "no per-step check" + ("" if r.get("params_in_sync", True) else " (final parameters DIFFER)")
    grad, param = r.get("first_gradient_difference"), r.get("first_parameter_difference")
    if grad is not None and (param is None or grad <= param):
        return "gradients differ after all_reduce"
    if param is not None:
        return "parameters differ, gradients equal"
    return "in sync" if r.get("params_in_sync", True) else "final parameters differ, per-step checks clean"


def ddp_report(paths, out: Path | None) -> int:
    runs = records(paths, lambda d: "params_in_sync" in d and "samples_per_sec" in d)
    if not runs:
        print("no train_synthetic records found")
        return 2
    lines = ["# Data-parallel runs: did the replicas stay identical?", "",
             "| run | ranks | engine | compression | samples/s | first gradient difference | "
             "first parameter difference | verdict |", "|---|---|---|---|---|---|---|---|"]
    bad = 0
    for name, r in runs:
        verdict = ddp_verdict(r)
        bad += verdict != "in sync" and not verdict.startswith("no per-step check")
        env = (r.get("environment") or {}).get("env") or {}
        show = lambda v: "-" if v is None else f"step {v}"          # noqa: E731
        lines.append(f"| {name} | {r.get('world_size')} | {r.get('engine', '-')} | "
                     f"{env.get('GPUBRIDGE_BRIDGE_COMPRESSION') or '-'} | {r['samples_per_sec']} | "
                     f"{show(r.get('first_gradient_difference'))} | {show(r.get('first_parameter_difference'))} | "
                     f"{verdict} |")
    lines += ["", f"{len(runs) - bad} of {len(runs)} runs in sync."]
    text = "\n".join(lines) + "\n"
    if out is not None:
        out.mkdir(parents=True, exist_ok=True)
        (out / "train_ddp_report.md").write_text(text)
    print(text, end="")
    return 1 if bad else 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    sub = ap.add_subparsers(dest="what", required=True)
    dp = sub.add_parser("dp")
    dp.add_argument("paths", nargs="+", type=Path)
    dp.add_argument("--out", type=Path, required=True)
    dp.add_argument("--baseline", type=Path)
    dp.add_argument("--tail", type=int, default=100)
    ddp = sub.add_parser("ddp")
    ddp.add_argument("paths", nargs="+", type=Path)
    ddp.add_argument("--out", type=Path)
    args = ap.parse_args(argv)
    if args.what == "dp":
        return dp_report(args.paths, args.out, args.baseline, args.tail)
    return ddp_report(args.paths, args.out)


if __name__ == "__main__":
    sys.exit(main())
