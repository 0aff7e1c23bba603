"""Prove that the stream-ordering tests have teeth.  Needs one GPU.

    python -m gpubridge_b200.kit.stream_mutations --out DIR [--mutation NAME ...] [--list]

Every switch of :mod:`gpubridge_b200._mutation` removes one stream-to-stream wait, and
``tests/test_gpu_streams.py`` pairs it with the test that guards that wait.  This program
runs each pair as an *experiment* - the guarding test in a fresh pytest process with the
switch on - and then one *control*: all guarding tests with no switch.  Outcomes are read
from pytest's JUnit report (one ``<testcase>`` per test), not from its console text:

* an experiment passes the audit when its test FAILED and the failure message counts wrong
  elements (the test saw stale or poisoned data - not a crash, not a timeout);
* the control passes when every test passed.

``report.json`` in ``--out`` lists every run with its verdict.  Exit status: 0 all verdicts
good, 1 some switch went unnoticed (or the control failed), 2 nothing ran (no GPU: every test
was skipped).
"""
from __future__ import annotations

import argparse
import dataclasses
import json
import os
import subprocess
import sys
import tempfile
import time
import xml.etree.ElementTree as ElementTree
from pathlib import Path

ROOT = Path(__file__).resolve().parents[2]
TEST_FILE = ROOT / "tests" / "test_gpu_streams.py"
SWITCH_ENV = "GPUBRIDGE_TEST_MUTATION"
WRONG_VALUES = "elements wrong"            # how test_gpu_streams.py words a data mismatch


def pairs() -> dict[str, str]:
    """switch -> name of the test that guards the wait it removes (read from the test file's
    ``MUTATIONS`` table without importing torch-heavy fixtures twice)."""
    scope: dict = {}
    source = TEST_FILE.read_text()
    start = source.index("MUTATIONS = {")
    depth, end = 0, start
    for end in range(source.index("{", start), len(source)):
        depth += {"{": 1, "}": -1}.get(source[end], 0)
        if depth == 0:
            break
    exec(source[start:end + 1], scope)  # noqa: S102 - our own test file's literal table
    return {switch: test for switch, (_, test) in scope["MUTATIONS"].items()}


@dataclasses.dataclass
class Run:
    """One pytest process and what became of its tests."""
    switch: str | None
    tests: list[str]
    seconds: float = 0.0
    outcomes: dict[str, str] = dataclasses.field(default_factory=dict)     # test -> passed/failed/skipped/error
    messages: list[str] = dataclasses.field(default_factory=list)
    timed_out: bool = False

    def command(self, report: Path | str) -> list[str]:
        selection = [f"{TEST_FILE}::{name}" for name in self.tests]
        return [sys.executable, "-m", "pytest", "-m", "gpu", "-q", "-p", "no:cacheprovider",
                f"--junitxml={report}", *selection]

    def execute(self, limit: float) -> None:
        env = dict(os.environ)
        env.pop(SWITCH_ENV, None)
        if self.switch:
            env[SWITCH_ENV] = self.switch
        with tempfile.TemporaryDirectory() as scratch:
            report = Path(scratch) / "junit.xml"
            began = time.monotonic()
            try:
                subprocess.run(self.command(report), cwd=ROOT, env=env, capture_output=True,
                               text=True, timeout=limit)
            except subprocess.TimeoutExpired:
                self.timed_out = True
            self.seconds = round(time.monotonic() - began, 1)
            if report.exists():
                self._read(report)

    def _read(self, report: Path) -> None:
        for case in ElementTree.parse(report).getroot().iter("testcase"):
            name, outcome = case.get("name", "?"), "passed"
            for child in case:
                if child.tag in ("failure", "error", "skipped"):
                    outcome = {"failure": "failed"}.get(child.tag, child.tag)
                    text = f"{child.get('message', '')} {child.text or ''}"
                    for line in text.splitlines():
                        if WRONG_VALUES in line or outcome == "error":
                            self.messages.append(line.strip()[:200])
                            break
            self.outcomes[name] = outcome

    @property
    def verdict(self) -> str:
        seen = set(self.outcomes.values())
        if self.timed_out:
            return "timed out"
        if not self.outcomes or seen == {"skipped"}:
            return "did not run"
        if "error" in seen:
            return "broken (set-up or collection error)"
        if self.switch is None:
            return "clean run passes" if seen == {"passed"} else "clean run FAILS"
        if "failed" not in seen:
            return "UNNOTICED"
        saw_data = any(WRONG_VALUES in m for m in self.messages)
        return "noticed" if saw_data else "failed for another reason"

    @property
    def good(self) -> bool:
        return self.verdict in ("noticed", "clean run passes")


def main(argv: list[str] | None = None) -> int:
    table = pairs()
    parser = argparse.ArgumentParser(description="Audit the stream-ordering tests with the mutation switches.")
    parser.add_argument("--out", type=Path, default=ROOT / "results" / "stream_mutations")
    parser.add_argument("--mutation", action="append", choices=sorted(table), help="audit only this switch")
    parser.add_argument("--timeout", type=float, default=600, help="seconds per pytest process")
    parser.add_argument("--list", "--dry-run", dest="list_only", action="store_true",
                        help="print the commands and stop")
    args = parser.parse_args(argv)
    switches = args.mutation or list(table)
    runs = [Run(switch, [table[switch]]) for switch in switches]
    runs.append(Run(None, sorted({table[s] for s in switches})))
    if args.list_only:
        for run in runs:
            setting = f"{SWITCH_ENV}={run.switch} " if run.switch else ""
            print("+ " + setting + " ".join(run.command("junit.xml")))
        return 0
    for run in runs:
        run.execute(args.timeout)
        label = run.switch or "(control: no switch)"
        print(f"{label:<26} {run.verdict:<34} {run.seconds:>6.1f} s  {', '.join(run.tests)}", flush=True)
    args.out.mkdir(parents=True, exist_ok=True)
    (args.out / "report.json").write_text(json.dumps(
        [dict(dataclasses.asdict(run), verdict=run.verdict) for run in runs], indent=2))
    if all(run.verdict == "did not run" for run in runs):
        print("no test ran: is a GPU visible?")
        return 2
    ok = all(run.good for run in runs)
    print("audit passed: every removed wait was noticed as wrong data, and the control is clean"
          if ok else "audit FAILED: see the verdicts above")
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
