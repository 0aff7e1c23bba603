"""What ``import gpubridge_b200`` costs on top of ``import torch``.

    python -m gpubridge_b200.bench.bench_import [--runs 5] [--out import.json]

Each run is a fresh interpreter: one that imports torch and torch.distributed only, one that
imports the package as well; the difference of the medians is the package's own import time
(it imports no kernels, builds nothing and touches no GPU until ``init()``).  Also lists the
package's modules that took longest (``-X importtime``).  Counterpart of the reference's
``scripts/bench_import.py``.
"""
from __future__ import annotations

import argparse
import json
import statistics
import subprocess
import sys
import time
from pathlib import Path

BASE = "import torch, torch.distributed"
OURS = BASE + "; import gpubridge_b200"


def seconds(code: str) -> float:
    t0 = time.perf_counter()
    subprocess.run([sys.executable, "-c", code], check=True, capture_output=True)
    return time.perf_counter() - t0


def slowest_modules(top: int) -> list[dict]:
    done = subprocess.run([sys.executable, "-X", "importtime", "-c", OURS], capture_output=True, text=True)
    rows = []
    for line in done.stderr.splitlines():
        # "import time:      self |  cumulative | package.module"
        parts = line.removeprefix("import time:").split("|")
        if len(parts) == 3 and parts[2].strip().startswith("gpubridge_b200"):
            rows.append({"module": parts[2].strip(), "self_ms": int(parts[0]) / 1e3,
                         "cumulative_ms": int(parts[1]) / 1e3})
    return sorted(rows, key=lambda r: -r["self_ms"])[:top]


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--runs", type=int, default=5)
    ap.add_argument("--top", type=int, default=8)
    ap.add_argument("--out", type=Path)
    args = ap.parse_args(argv)
    seconds(BASE)                                         # page the libraries in once
    base, ours = [], []
    for _ in range(args.runs):                            # interleaved: drift hits both alike
        base.append(seconds(BASE))
        ours.append(seconds(OURS))
    record = {"runs": args.runs, "torch_only_s": round(statistics.median(base), 3),
              "with_package_s": round(statistics.median(ours), 3),
              "package_ms": round((statistics.median(ours) - statistics.median(base)) * 1e3, 1),
              "slowest_modules": slowest_modules(args.top)}
    print(f"import torch: {record['torch_only_s']} s; with gpubridge_b200: {record['with_package_s']} s; "
          f"the package adds {record['package_ms']} ms")
    for row in record["slowest_modules"]:
        print(f"  {row['self_ms']:7.1f} ms  {row['module']}")
    if args.out:
        args.out.parent.mkdir(parents=True, exist_ok=True)
        args.out.write_text(json.dumps(record, indent=1))
    return 0


if __name__ == "__main__":
    sys.exit(main())
