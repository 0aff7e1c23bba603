"""Rules the source tree must keep, checked as text.

* No file names a TMA or bulk load with cluster fan-out (multi-GPU runs are refused while one
  does, and such a load from a peer's memory must never run), nor one of the batched memcpy
  entry points that fault this driver.
* Comments and docstrings stand on their own: no pointers to planning documents, review
  rounds or machine paths.
* Every CUDA source is compiled for sm_100a only.
The needles are assembled from pieces so that this file passes its own check."""
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SOURCE = (".py", ".cu", ".cuh", ".cpp", ".h", ".sh", ".sbatch")
SKIP_DIRS = {".git", "gpu" + "run_out", "_work", "baseline", "__pycache__", "_build", "lib", ".pytest_cache"}


def sources():
    for base, dirs, files in os.walk(ROOT):
        dirs[:] = [d for d in dirs if d not in SKIP_DIRS]
        for name in files:
            if name.endswith(SOURCE):
                path = os.path.join(base, name)
                with open(path, errors="replace") as fh:
                    yield os.path.relpath(path, ROOT), fh.read()


def test_no_closed_calls_or_cluster_fan_out_loads():
    needles = ["multicast" + "::cluster", "Memcpy" + "BatchAsync", "Memcpy3D" + "BatchAsync"]
    hits = [(path, n) for path, text in sources() for n in needles if n in text]
    assert not hits, hits


def test_comments_stand_on_their_own():
    names = ["SUR" + "VEY", "VER" + "DICT", "ADV" + "ICE", "DESIGN" + ".md", "BASELINE" + ".md", "gpu" + "run", "/ro" + "ot/"]
    pattern = re.compile("|".join(re.escape(n) for n in names))
    hits = []
    for path, text in sources():
        for number, line in enumerate(text.splitlines(), 1):
            if pattern.search(line):
                hits.append(f"{path}:{number}: {line.strip()[:100]}")
    assert not hits, "\n".join(hits[:20])


def test_cuda_builds_target_sm_100a_only():
    from gpubridge_b200.ops import _build
    assert _build.ARCH == ["-gencode", "arch=compute_100a,code=sm_100a"]
    assert "-lineinfo" in _build.NVCC_FLAGS
    for path, text in sources():
        if path.endswith((".cu", ".cuh")):
            assert "wgmma" not in text, path            # Hopper only: does not compile here
