"""The validation kit on a rented notebook machine: one to eight B200s, a shell, nothing set up.

    python notebook.py --source https://example.org/gpubridge-b200.git --ref v0.2 --work /tmp/gb
    python notebook.py --source /path/to/checkout --only features gpu_tests
    python notebook.py --dry-run
    python notebook.py --write-notebook kit.ipynb        # the same steps, one cell each

The file runs on its own (standard library only) until the package under test has been
fetched, so it can be pasted into a notebook's first cell.  Steps, in order:

``fetch``      the package under test: ``git clone --branch REF`` of a URL, or a copy of a
               local checkout, into ``<work>/src`` (outside the results, which are what a
               notebook saves);
``build``      the native library and the C++ front end, in-tree (nvcc for sm_100a);
``versions``   nvidia-smi, torch, CUDA, NCCL versions -> ``versions.json``;
``features``   what this machine can run, each probed in a child: CUDA events, bf16 matrix
               products, compute capability 10.0 (tcgen05 kernels), peer access between GPUs,
               NVLink multicast (in-switch reduction); a later step that needs a missing
               feature is skipped and the journal says why;
``gpu_tests``  ``pytest -m gpu``;
``runbook``    the one-box runbook (:mod:`gpubridge_b200.kit.runbook`): checks per island
               split and policy, negative init, p2p, numerical gate, stream mutations, a
               sweep against NCCL, weak scaling;
``codec``      the codec kernels against the CPU oracle and their bandwidth;
``fsdp2``      the FSDP2 example across two islands with ``--verify``;
``tables``     the validation tables over everything above;
``package``    one ``.tar.gz`` of the results directory.

Every step is a child process group under a hard limit; one that fails or runs over is
recorded and the rest still run.  ``steps.jsonl`` has the kit's usual rows (the reference runs
its kit the same way on a free two-GPU notebook: scripts/gpu/kaggle/kaggle_gpubridge.py).
"""
from __future__ import annotations

import argparse
import json
import os
import shutil
import signal
import subprocess
import sys
import tarfile
import time
from pathlib import Path

STEPS = ("fetch", "build", "versions", "features", "gpu_tests", "runbook", "codec", "fsdp2",
         "tables", "package")
LIMITS = {"fetch": 300, "build": 1800, "versions": 120, "features": 600, "gpu_tests": 2400,
          "runbook": 7200, "codec": 900, "fsdp2": 900, "tables": 300, "package": 300}
#: feature -> a program that exits 0 when the machine has it
PROBES = {
    "cuda_events": "import torch; a=torch.cuda.Event(enable_timing=True); b=torch.cuda.Event(enable_timing=True);"
                   " a.record(); torch.ones(8, device='cuda').sum(); b.record(); b.synchronize(); a.elapsed_time(b)",
    "bf16_matmul": "import torch; x=torch.ones(64, 64, device='cuda', dtype=torch.bfloat16);"
                   " assert float((x @ x)[0, 0]) == 64.0",
    "sm_100": "import torch; assert torch.cuda.get_device_capability(0) == (10, 0)",
    "two_gpus": "import torch; assert torch.cuda.device_count() >= 2",
    "peer_access": "import torch; assert torch.cuda.device_count() >= 2 and torch.cuda.can_device_access_peer(0, 1)",
    "multicast": "from gpubridge_b200.ops import switch, _lib; assert switch.supported(_lib.lib(), 0)",
}
#: step -> features it cannot run without
NEEDS = {"gpu_tests": ("sm_100",), "runbook": ("sm_100", "cuda_events"), "codec": ("sm_100",),
         "fsdp2": ("sm_100", "two_gpus", "peer_access")}


class Runner:
    def __init__(self, work: Path, out: Path, source: str, ref: str, python: str = sys.executable,
                 limits: dict | None = None, run=None) -> None:
        self.work, self.out, self.source, self.ref, self.python = work, out, source, ref, python
        self.src = work / "src"
        self.limits = dict(LIMITS, **(limits or {}))
        self.features: dict[str, bool] = {}
        self._run = run or self._child

    # -- children -------------------------------------------------------------------------------------
    def _child(self, cmd: list[str], limit: float, log: Path, env: dict | None = None) -> int | None:
        """Run ``cmd`` as its own process group; past ``limit`` seconds the whole group is
        killed.  Returns the exit code, None when the limit was hit."""
        full = dict(os.environ, PYTHONPATH=os.pathsep.join(
            filter(None, [str(self.src), os.environ.get("PYTHONPATH", "")])), **(env or {}))
        with open(log, "ab") as sink:
            child = subprocess.Popen(cmd, stdout=sink, stderr=subprocess.STDOUT, env=full,
                                     cwd=str(self.src if self.src.exists() else self.work),
                                     start_new_session=True)
            try:
                return child.wait(timeout=limit)
            except subprocess.TimeoutExpired:
                os.killpg(child.pid, signal.SIGKILL)
                child.wait()
                return None

    def commands(self, step: str) -> list[list[str]]:
        py, out = self.python, self.out
        if step == "fetch":
            if Path(self.source).exists():
                return [[py, "-c", "import shutil, sys; shutil.copytree(sys.argv[1], sys.argv[2], "
                         "dirs_exist_ok=True, ignore=shutil.ignore_patterns('.git', '__pycache__', '*.o'))",
                         self.source, str(self.src)]]
            return [["git", "clone", "--depth", "1", *(["--branch", self.ref] if self.ref else []),
                     self.source, str(self.src)]]
        if step == "build":
            return [[py, "-c", "import __graft_entry__ as entry; entry.build()"]]
        if step == "versions":
            return [[py, "-c", "import json, subprocess, sys, torch; json.dump({'torch': torch.__version__, "
                     "'cuda': torch.version.cuda, 'nccl': '.'.join(map(str, torch.cuda.nccl.version())) "
                     "if torch.cuda.is_available() else None, 'gpus': [torch.cuda.get_device_name(i) for i in "
                     "range(torch.cuda.device_count())], 'nvidia_smi': subprocess.run(['nvidia-smi', '-L'], "
                     "capture_output=True, text=True).stdout.splitlines()}, open(sys.argv[1], 'w'), indent=1)",
                     str(out / "versions.json")]]
        if step == "gpu_tests":
            return [[py, "-m", "pytest", "tests", "-m", "gpu", "-q", "-rs"]]
        if step == "runbook":
            return [[py, "-m", "gpubridge_b200.kit.runbook", "--out", str(out / "runbook")]]
        if step == "codec":
            return [[py, "-m", "pytest", "tests/test_gpu_codec.py", "-q"],
                    [py, "-m", "gpubridge_b200.bench.bench_compression", "--numel", str(1 << 26)]]
        if step == "fsdp2":
            return [[py, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
                     "127.0.0.1", "--master-port", "29871", "examples/fsdp2_torch_backend.py", "--verify",
                     "--steps", "10", "--json", str(out / "fsdp2.json")]]
        if step == "tables":
            return [[py, "-m", "gpubridge_b200.kit.validation_tables", str(out), "--out", str(out / "tables.md")]]
        return []

    # -- steps ----------------------------------------------------------------------------------------
    def features_step(self, log: Path) -> tuple[bool, str]:
        for name, program in PROBES.items():
            code = self._run([self.python, "-c", program], 120, log)
            self.features[name] = code == 0
        (self.out / "features.json").write_text(json.dumps(self.features, indent=1))
        return True, ", ".join(f"{k}={'yes' if v else 'no'}" for k, v in self.features.items())

    def package_step(self) -> tuple[bool, str]:
        archive = self.work / f"{self.out.name}.tar.gz"
        with tarfile.open(archive, "w:gz") as tar:
            tar.add(self.out, arcname=self.out.name)
        return True, str(archive)

    def step(self, name: str) -> dict:
        log = self.out / f"{name}.log"
        started = time.monotonic()
        missing = [f for f in NEEDS.get(name, ()) if self.features and not self.features.get(f, False)]
        if missing:
            verdict, note = "skipped", f"this machine lacks {', '.join(missing)}"
        elif name == "features":
            ok, note = self.features_step(log)
            verdict = "ok" if ok else "failed"
        elif name == "package":
            ok, note = self.package_step()
            verdict = "ok"
        else:
            verdict, note = "ok", ""
            for cmd in self.commands(name):
                code = self._run(cmd, self.limits[name], log)
                if code is None:
                    verdict, note = "timeout", f"killed after {self.limits[name]} s"
                    break
                if code != 0:
                    verdict, note = "failed", f"exit code {code}"
                    break
        row = {"step": name, "verdict": verdict, "ok": verdict in ("ok", "skipped"), "note": note,
               "seconds": round(time.monotonic() - started, 1), "log": log.name}
        with open(self.out / "steps.jsonl", "a") as journal:
            journal.write(json.dumps(row) + "\n")
        return row


def notebook(steps, source: str, ref: str) -> dict:
    """The same run as a notebook: the first cell holds this file, then one cell per step."""
    here = Path(__file__).read_text()

    def cell(text: str) -> dict:
        return {"cell_type": "code", "metadata": {}, "execution_count": None, "outputs": [],
                "source": text.splitlines(keepends=True)}

    cells = [{"cell_type": "markdown", "metadata": {}, "source": [
        "# gpubridge-b200 validation kit\n", "Run the cells in order; each step is limited in time and a "
        "failed one does not stop the rest.  Download the archive the last cell names.\n"]},
        cell("%%writefile notebook_kit.py\n" + here)]
    for name in steps:
        ref_flag = f" --ref {ref}" if ref else ""
        cells.append(cell(f"!python notebook_kit.py --source {source}{ref_flag} --only {name}"))
    return {"cells": cells, "metadata": {"kernelspec": {"display_name": "Python 3", "language": "python",
                                                        "name": "python3"}},
            "nbformat": 4, "nbformat_minor": 5}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--source", default=str(Path(__file__).resolve().parents[2]),
                    help="git URL or local checkout of the package under test")
    ap.add_argument("--ref", default="", help="tag or branch to clone")
    ap.add_argument("--work", type=Path, default=Path("/tmp/gpubridge-b200-kit"))
    ap.add_argument("--only", nargs="*", default=None)
    ap.add_argument("--dry-run", action="store_true")
    ap.add_argument("--write-notebook", type=Path)
    args = ap.parse_args(argv)
    steps = [s for s in STEPS if not args.only or s in args.only]
    unknown = set(args.only or ()) - set(STEPS)
    if unknown:
        ap.error(f"unknown steps: {', '.join(sorted(unknown))}; known: {', '.join(STEPS)}")
    if args.write_notebook:
        args.write_notebook.write_text(json.dumps(notebook(steps, args.source, args.ref), indent=1))
        print(args.write_notebook)
        return 0
    out = args.work / "results"
    runner = Runner(args.work, out, args.source, args.ref)
    if args.dry_run:
        for name in steps:
            print(f"[{name}] limit {runner.limits[name]} s")
            for cmd in runner.commands(name):
                print("  + " + " ".join(cmd)[:200])
        return 0
    out.mkdir(parents=True, exist_ok=True)
    known = out / "features.json"
    if known.exists() and "features" not in steps:
        runner.features = json.loads(known.read_text())
    failed = []
    for name in steps:
        print(f"[kit] {name} ...", end=" ", flush=True)
        row = runner.step(name)
        print(f"{row['verdict']} ({row['seconds']} s) {row['note']}", flush=True)
        if not row["ok"]:
            failed.append(name)
    print("every step passed" if not failed else f"failed steps: {', '.join(failed)}")
    return 1 if failed else 0


if __name__ == "__main__":
    sys.exit(main())
