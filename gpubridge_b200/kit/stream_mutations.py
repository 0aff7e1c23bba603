"""Show that the GPU stream-ordering tests catch what they guard.  Needs one GPU.

    python -m gpubridge_b200.kit.stream_mutations --out results/stream_mutations [--mutation NAME]

``tests/test_gpu_streams.py`` names, for every switch in ``gpubridge_b200._mutation``, the test
that guards the stream-to-stream wait the switch removes.  Each guarded test is run with its
switch on (``GPUBRIDGE_TEST_MUTATION``): it must fail, and on wrong values, not by crashing.
Then all of them run without a switch and must pass.  Writes ``mutations.json``; exit code 0
only if every mutation was caught and the clean run passed, 2 if the tests did not run (no
GPU).  Same procedure as the reference's ``scripts/gpu/stream_mutations.py``.
"""
from __future__ import annotations

import argparse
import importlib.util
import json
import os
import re
import subprocess
import sys
import time
from pathlib import Path

REPO = Path(__file__).resolve().parents[2]
TESTS = REPO / "tests" / "test_gpu_streams.py"
COUNTS = re.compile(r"\b(\d+) (passed|failed|skipped|errors?|deselected)\b")


def guarded() -> dict[str, str]:
    spec = importlib.util.spec_from_file_location("stream_tests_for_mutations", TESTS)
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return {name: test for name, (_, test) in module.MUTATIONS.items()}


def pytest_command(tests: list[str]) -> list[str]:
    return [sys.executable, "-m", "pytest", "-m", "gpu", str(TESTS), "-q", "-p",
            "no:cacheprovider", "-k", " or ".join(tests)]


def run(tests: list[str], mutation: str | None, timeout: float) -> dict:
    env = {k: v for k, v in os.environ.items() if k != "GPUBRIDGE_TEST_MUTATION"}
    if mutation:
        env["GPUBRIDGE_TEST_MUTATION"] = mutation
    t0 = time.monotonic()
    try:
        done = subprocess.run(pytest_command(tests), cwd=REPO, env=env, capture_output=True,
                              text=True, timeout=timeout)
        text, code = done.stdout + done.stderr, done.returncode
    except subprocess.TimeoutExpired as exc:
        text, code = f"{exc.stdout or ''}{exc.stderr or ''}\nran past {timeout:g} s", None
    counts = {kind.rstrip("s"): int(n) for n, kind in COUNTS.findall(text)}
    evidence = [line.strip() for line in text.splitlines()
                if re.search(r"elements wrong|Error|FAILED", line)]
    wrong = [line for line in evidence if "elements wrong" in line]
    return {"tests": tests, "mutation": mutation, "exit_code": code, "counts": counts,
            "seconds": round(time.monotonic() - t0, 1), "wrong_values": bool(wrong),
            "evidence": (wrong or evidence)[:8]}


def main(argv=None) -> int:
    known = guarded()
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--out", type=Path, default=REPO / "results" / "stream_mutations")
    ap.add_argument("--mutation", action="append", choices=sorted(known))
    ap.add_argument("--timeout", type=float, default=600)
    ap.add_argument("--dry-run", action="store_true")
    args = ap.parse_args(argv)
    chosen = args.mutation or list(known)
    plan = [(name, [known[name]]) for name in chosen]
    plan.append((None, sorted({known[name] for name in chosen})))
    if args.dry_run:
        for mutation, tests in plan:
            prefix = f"GPUBRIDGE_TEST_MUTATION={mutation} " if mutation else ""
            print(f"+ {prefix}{' '.join(pytest_command(tests))}")
        return 0
    rows = []
    for mutation, tests in plan:
        row = run(tests, mutation, args.timeout)
        ran = row["counts"].get("passed", 0) + row["counts"].get("failed", 0)
        if row["exit_code"] is None:
            row["verdict"] = "timed out"
        elif row["counts"].get("error"):
            row["verdict"] = "error (collection or set-up)"
        elif not ran:
            row["verdict"] = "did not run (no GPU?)"
        elif mutation and row["counts"].get("failed"):
            row["verdict"] = "caught" if row["wrong_values"] else "failed, but not on wrong values"
        elif mutation:
            row["verdict"] = "NOT CAUGHT"
        else:
            row["verdict"] = "passed" if not row["counts"].get("failed") else "FAILED"
        rows.append(row)
        print(f"{mutation or 'no mutation':<24} {', '.join(tests)}: {row['verdict']} "
              f"({row['seconds']} s)", flush=True)
    args.out.mkdir(parents=True, exist_ok=True)
    (args.out / "mutations.json").write_text(json.dumps(rows, indent=2))
    if any(r["verdict"].startswith("did not run") for r in rows):
        return 2
    good = all(r["verdict"] in ("caught", "passed") for r in rows)
    print("every mutation was caught and the clean run passes" if good else
          "a mutation went uncaught, or the clean run fails (see above)")
    return 0 if good else 1


if __name__ == "__main__":
    sys.exit(main())
