"""Which build produced a number: one JSON record to keep beside every benchmark result.

    python -m gpubridge_b200.kit.baseline_identity OUT.json

A benchmark row is only comparable with another when both were made by the same sources,
the same compiler and the same libraries, and an identical commit can hide a difference in
any of the three (a stale ``.so``, another torch wheel, another nvcc).  So everything here is
read from what is actually installed and built, never assumed:

* ``source``: git commit and dirty flag, and a SHA-256 over the tracked content of every
  source tree (``csrc``, ``csrc_torch``, the Python package, ``tests``, ``bench.py``);
* ``native``: name, size and SHA-256 of every library the tree built (the kernels' library,
  the C++ ``torch.distributed`` front end) and whether the kernels' library is older than
  its sources;
* ``toolchain``: nvcc, the host compiler, the CUDA runtime and NCCL torch was built against;
* ``packages``: versions of the Python packages a result depends on;
* ``reference``: the same for the reference build under ``baseline/_ref`` when it is there
  (its version and a hash of its sources), so both arms of a comparison are pinned;
* ``environment``: the kit's own record of this process (devices, probe, redacted variables).

Counterpart of the reference's scripts/baseline_identity.py.
"""
from __future__ import annotations

import hashlib
import json
import platform
import shutil
import subprocess
import sys
from importlib import metadata
from pathlib import Path

ROOT = Path(__file__).resolve().parents[2]
PACKAGES = ("torch", "numpy", "triton", "pytest", "pytest-timeout", "nvidia-nccl-cu12", "pybind11")
TREES = ("gpubridge_b200/csrc", "gpubridge_b200/csrc_torch", "gpubridge_b200", "tests", "bench.py")
SUFFIXES = (".py", ".cu", ".cuh", ".cpp", ".h", ".sh", ".sbatch", ".toml")


def run(*command: str) -> str | None:
    """Stdout of a command, or None when it is absent or fails."""
    if shutil.which(command[0]) is None:
        return None
    try:
        done = subprocess.run(command, capture_output=True, text=True, cwd=ROOT, timeout=60)
    except (OSError, subprocess.SubprocessError):
        return None
    return done.stdout.strip() if done.returncode == 0 else None


def tree_digest(path: Path) -> dict | None:
    """Files and a SHA-256 over names and contents of the sources under ``path`` (build output
    and caches left out), so two checkouts can be compared without git."""
    if not path.exists():
        return None
    files = [path] if path.is_file() else sorted(
        p for p in path.rglob("*") if p.is_file() and p.suffix in SUFFIXES
        and not {"_build", "lib", "__pycache__"} & set(p.relative_to(path).parts))
    digest = hashlib.sha256()
    for file in files:
        digest.update(str(file.relative_to(ROOT)).encode() + b"\0" + file.read_bytes() + b"\0")
    return {"files": len(files), "sha256": digest.hexdigest()}


def library(path: Path) -> dict | None:
    if not path.exists():
        return None
    return {"name": path.name, "bytes": path.stat().st_size,
            "sha256": hashlib.sha256(path.read_bytes()).hexdigest(),
            "modified": int(path.stat().st_mtime)}


def version_of(package: str) -> str | None:
    try:
        return metadata.version(package)
    except metadata.PackageNotFoundError:
        return None


def identity() -> dict:
    import torch
    from gpubridge_b200 import kit
    from gpubridge_b200.ops import _build, _build_c10d
    kernels = Path(_build.LIB)
    newest_source = max((p.stat().st_mtime for p in Path(_build.CSRC).iterdir() if p.is_file()), default=0)
    reference = ROOT / "baseline" / "_ref" / "gpubridge"
    record = {
        "source": {"commit": run("git", "rev-parse", "HEAD"),
                   "dirty": bool(run("git", "status", "--porcelain")),
                   "trees": {tree: tree_digest(ROOT / tree) for tree in TREES}},
        "native": {"kernels": library(kernels), "front_end": library(Path(_build_c10d.OUT)),
                   "kernels_older_than_sources": kernels.exists() and kernels.stat().st_mtime < newest_source,
                   "front_end_stale": _build_c10d.stale(),
                   "flags": " ".join(_build.ARCH + _build.NVCC_FLAGS)},
        "toolchain": {"nvcc": (run("nvcc", "--version") or "").splitlines()[-1:] or None,
                      "cxx": (run("c++", "--version") or "").splitlines()[:1] or None,
                      "torch_cuda": torch.version.cuda,
                      "nccl": ".".join(map(str, torch.cuda.nccl.version())) if torch.cuda.is_available() else None,
                      "python": platform.python_version(), "machine": platform.machine()},
        "packages": {name: version_of(name) for name in PACKAGES},
        "reference": {"installed": reference.is_dir(), "version": version_of("gpubridge"),
                      "tree": tree_digest(reference) if reference.is_dir() else None},
        "environment": kit.environment(),
    }
    return record


def main(argv: list[str] | None = None) -> int:
    argv = sys.argv[1:] if argv is None else argv
    if argv and argv[0] in ("-h", "--help"):
        print(__doc__)
        return 0
    if len(argv) != 1 or argv[0].startswith("-"):
        print("usage: python -m gpubridge_b200.kit.baseline_identity OUT.json", file=sys.stderr)
        return 2
    out = Path(argv[0])
    out.parent.mkdir(parents=True, exist_ok=True)
    out.write_text(json.dumps(identity(), indent=2, default=str))
    print(out)
    return 0


if __name__ == "__main__":
    sys.exit(main())
