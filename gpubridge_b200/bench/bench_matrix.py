"""The comparison matrix: several all-reduce sweeps side by side.

    python -m gpubridge_b200.bench.bench_matrix one-island=sweep8_none.json islands-4+4=sweep8_44.json \\
        [--baseline one-island/nccl] [--out DIR]

Each argument names a run and the JSON a ``bench_all_reduce --json`` sweep wrote; a run
contributes one column per target it measured (``ours``, ``nccl``, ``policy:...``,
``compression:...``).  For three size ranges (under 256 KB, 256 KB to under 64 MB, 64 MB and
up) the table gives every column's median latency, bus bandwidth and time as a multiple of
the baseline column at the same size (default: the first ``nccl`` column).  Writes
``matrix.md``, ``matrix.json`` and ``matrix.csv``.  Counterpart of the reference's
``scripts/gpu/bench_matrix.py`` (its runs differ by machine pair; here they differ by island
split, policy and compression on one box).
"""
from __future__ import annotations

import argparse
import csv
import json
import statistics
import sys
from pathlib import Path

RANGES = (("under 256 KB", 0, 256 << 10), ("256 KB to under 64 MB", 256 << 10, 64 << 20),
          ("64 MB and up", 64 << 20, 1 << 62))


def load(path: Path) -> dict[str, dict[int, dict]]:
    """{target: {bytes: row}} of one sweep file (all_reduce rows of the first dtype)."""
    data = json.loads(path.read_text())
    rows = data["rows"] if isinstance(data, dict) else data
    out: dict[str, dict[int, dict]] = {}
    for r in rows:
        if r.get("op", "all_reduce") != "all_reduce":
            continue
        out.setdefault(r["target"], {})[int(r["bytes"])] = r
    return out


def human(n: int) -> str:
    for unit, size in (("G", 1 << 30), ("M", 1 << 20), ("K", 1 << 10)):
        if n >= size and n % size == 0:
            return f"{n // size}{unit}"
    return str(n)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("runs", nargs="+", metavar="NAME=FILE")
    ap.add_argument("--baseline", default="")
    ap.add_argument("--out", type=Path, default=None)
    args = ap.parse_args(argv)
    columns: dict[str, dict[int, dict]] = {}
    for item in args.runs:
        name, _, path = item.partition("=")
        if not path:
            ap.error(f"{item!r}: expected NAME=FILE")
        for target, rows in load(Path(path)).items():
            columns[f"{name}/{target}"] = rows
    if not columns:
        ap.error("no all_reduce rows in the given files")
    baseline = args.baseline or next((c for c in columns if c.endswith("/nccl")), next(iter(columns)))
    if baseline not in columns:
        ap.error(f"baseline {baseline!r} is not one of {sorted(columns)}")
    sizes = sorted({b for rows in columns.values() for b in rows})
    table, lines = [], [f"# All-reduce matrix (baseline: `{baseline}`)", ""]
    for label, lo, hi in RANGES:
        picked = [b for b in sizes if lo <= b < hi]
        if not picked:
            continue
        lines += [f"## {label}", "",
                  "| size | " + " | ".join(f"{c} us (GB/s, x baseline)" for c in columns) + " |",
                  "|---|" + "---|" * len(columns)]
        for b in picked:
            base = columns[baseline].get(b)
            cells = []
            for name, rows in columns.items():
                r = rows.get(b)
                if r is None:
                    cells.append("-")
                    continue
                ratio = r["ms"] / base["ms"] if base else None
                cells.append(f"{r['ms'] * 1e3:.1f} ({r['busbw_gbs']:.1f}"
                             + (f", {ratio:.2f}x" if ratio is not None else "") + ")")
                table.append({"range": label, "bytes": b, "column": name, "us": round(r["ms"] * 1e3, 2),
                              "busbw_gbs": r["busbw_gbs"],
                              "times_baseline": round(ratio, 3) if ratio is not None else None})
            lines.append(f"| {human(b)} | " + " | ".join(cells) + " |")
        lines.append("")
        summary = []
        for name in columns:
            ratios = [t["times_baseline"] for t in table
                      if t["range"] == label and t["column"] == name and t["times_baseline"]]
            if ratios:
                summary.append(f"`{name}` {statistics.median(ratios):.2f}x")
        lines += ["Median time as a multiple of the baseline: " + ", ".join(summary) + ".", ""]
    text = "\n".join(lines) + "\n"
    print(text)
    out = args.out
    if out is not None:
        out.mkdir(parents=True, exist_ok=True)
        (out / "matrix.md").write_text(text)
        (out / "matrix.json").write_text(json.dumps({"baseline": baseline, "rows": table}, indent=1))
        with open(out / "matrix.csv", "w", newline="") as fh:
            writer = csv.DictWriter(fh, fieldnames=list(table[0]))
            writer.writeheader()
            writer.writerows(table)
    return 0


if __name__ == "__main__":
    sys.exit(main())
