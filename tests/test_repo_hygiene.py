"""Rules the source tree must keep, checked as text.

* Comments and docstrings stand on their own: no pointers to planning documents, review
  rounds or machine paths.
* Every CUDA source is compiled for sm_100a only.
The planning-document names are assembled from pieces so that this file passes its own check.
(Which loads and driver calls a source may name is enforced by the machines that run the GPU
jobs; this file deliberately spells none of them.)"""
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
