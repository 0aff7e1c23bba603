"""Build the native library in-tree: ``gpubridge_b200/lib/libgpubridge_b200.so``.

Every ``.cu`` and ``.cpp`` under ``csrc/`` is compiled for sm_100a only
(``-gencode arch=compute_100a,code=sm_100a``) and linked into one shared library that the
Python side loads with ``ctypes``; the kernels take raw pointers and a ``cudaStream_t``,
so neither torch's headers nor pybind11 are involved and a full rebuild takes well under a
minute.  Objects are cached by source hash under ``gpubridge_b200/_build``.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(HERE)
CSRC = os.path.join(PKG, "csrc")
OBJ = os.path.join(PKG, "_build")
LIB_DIR = os.path.join(PKG, "lib")
LIB = os.path.join(LIB_DIR, "libgpubridge_b200.so")
LIB_BOUNDS = os.path.join(LIB_DIR, "libgpubridge_b200_bounds.so")

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-lineinfo", "-std=c++17", "--use_fast_math=false", "-Xcompiler", "-fPIC",
              "-Xcompiler", "-fvisibility=default", "--expt-relaxed-constexpr"]


def nvcc() -> str:
    for candidate in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if candidate and os.path.exists(candidate):
            return candidate
    raise RuntimeError("nvcc not found; the native library needs the CUDA 12.9 toolkit")


def sources() -> list[str]:
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cu", ".cpp")))


def _digest(path: str, extra: tuple[str, ...] = ()) -> str:
    h = hashlib.sha256()
    for name in sorted(os.listdir(CSRC)):
        if name.endswith((".cuh", ".h")) or os.path.join(CSRC, name) == path:
            with open(os.path.join(CSRC, name), "rb") as fh:
                h.update(name.encode() + b"\0" + fh.read())
    h.update(" ".join([*ARCH, *NVCC_FLAGS, *extra]).encode())
    return h.hexdigest()[:16]


def _compile(path: str, verbose: bool, extra: tuple[str, ...] = ()) -> str:
    obj = os.path.join(OBJ, f"{os.path.basename(path)}.{_digest(path, extra)}.o")
    if os.path.exists(obj):
        return obj
    flags = [f for f in NVCC_FLAGS if f != "--use_fast_math=false"] + list(extra)
    cmd = [nvcc(), *ARCH, *flags, "-I", CSRC, "-c", path, "-o", obj + ".tmp"]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    done = subprocess.run(cmd, capture_output=True, text=True)
    if done.returncode != 0:
        raise RuntimeError(f"nvcc failed for {path}:\n{done.stdout}\n{done.stderr}")
    if verbose:
        sys.stderr.write(done.stderr)
    os.replace(obj + ".tmp", obj)
    return obj


def build(verbose: bool = False, force: bool = False, bounds: bool = False) -> str:
    """Compile what changed and link the library; returns its path.  ``bounds``: the checked
    build (``-DGB_BOUNDS``: every access of the fabric kernels is compared with the ranges the
    host allowed), a second library beside the ordinary one."""
    os.makedirs(OBJ, exist_ok=True)
    os.makedirs(LIB_DIR, exist_ok=True)
    lib = LIB_BOUNDS if bounds else LIB
    extra = ("-DGB_BOUNDS",) if bounds else ()
    if force:
        for name in os.listdir(OBJ):
            if os.path.isfile(os.path.join(OBJ, name)):        # the front end's objects have a folder of their own
                os.remove(os.path.join(OBJ, name))
    with ThreadPoolExecutor(max_workers=4) as pool:
        objects = list(pool.map(lambda p: _compile(p, verbose, extra), sources()))
    stamp = os.path.join(OBJ, "linked_bounds.txt" if bounds else "linked.txt")
    keep = set(objects)
    for other in ("linked.txt", "linked_bounds.txt"):      # the other variant's objects stay
        other = os.path.join(OBJ, other)
        if other != stamp and os.path.exists(other):
            keep.update(open(other).read().split("\n"))
    for name in os.listdir(OBJ):               # objects of sources as they were before: dead weight
        path = os.path.join(OBJ, name)
        if name.endswith((".o", ".tmp")) and path not in keep:
            os.remove(path)
    want = "\n".join(objects)
    if os.path.exists(lib) and os.path.exists(stamp) and open(stamp).read() == want:
        return lib
    cmd = [nvcc(), *ARCH, "-shared", "-cudart", "shared", "-o", lib + ".tmp", *objects]
    done = subprocess.run(cmd, capture_output=True, text=True)
    if done.returncode != 0:
        raise RuntimeError(f"linking {lib} failed:\n{done.stdout}\n{done.stderr}")
    os.replace(lib + ".tmp", lib)
    with open(stamp, "w") as fh:
        fh.write(want)
    return lib


def main() -> int:
    """``python -m gpubridge_b200.ops._build [-v] [--force] [--bounds]``: build and print the path."""
    print(build(verbose="-v" in sys.argv, force="--force" in sys.argv, bounds="--bounds" in sys.argv))
    return 0


if __name__ == "__main__":
    sys.exit(main())
