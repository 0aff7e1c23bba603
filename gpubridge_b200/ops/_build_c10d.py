"""Build the C++ ``torch.distributed`` front end in-tree: ``gpubridge_b200/lib/gb_c10d.so``.

One host-only translation unit (``csrc_torch/gb_c10d.cpp``) against torch's headers, linked to
the native library beside it (``libgpubridge_b200.so``, found again at run time through an
``$ORIGIN`` rpath).  Kept apart from the main build because it is the only part that needs
torch's headers: the kernels build in seconds without them, this takes a minute or two.
"""
from __future__ import annotations

import importlib.util
import os
import sys

from gpubridge_b200.ops import _build

SRC = os.path.join(_build.PKG, "csrc_torch", "gb_c10d.cpp")
NAME = "gb_c10d"
OUT = os.path.join(_build.LIB_DIR, NAME + ".so")
WORK = os.path.join(_build.OBJ, "c10d")


STAMP = OUT + ".stamp"


def _digest() -> str:
    import hashlib
    h = hashlib.sha256()
    for path in (SRC, os.path.join(_build.CSRC, "gb_engine.h"), os.path.join(_build.CSRC, "gb_args.h")):
        with open(path, "rb") as fh:
            h.update(fh.read())
    import torch
    h.update(torch.__version__.encode())
    return h.hexdigest()[:16]


def stale() -> bool:
    """True when the module is missing or was built from other sources or another torch."""
    if not (os.path.exists(OUT) and os.path.exists(STAMP)):
        return True
    with open(STAMP) as fh:
        return fh.read().strip() != _digest()


def build(verbose: bool = False) -> str:
    """Compile when the source is newer than the module; returns the module's path."""
    if not stale() and os.path.exists(_build.LIB):
        return OUT                              # both libraries are there: nothing to compile
    _build.build()
    if not stale():
        return OUT
    from torch.utils import cpp_extension
    os.makedirs(WORK, exist_ok=True)
    # torch serialises builds of one directory with a lock FILE and waits for it without a
    # limit; a build that was killed (or a tree copied in mid-build) leaves it behind for ever
    lock = os.path.join(WORK, "lock")
    try:
        import time
        if time.time() - os.path.getmtime(lock) > 600:
            os.remove(lock)
    except OSError:
        pass
    cpp_extension.load(
        name=NAME, sources=[SRC], extra_include_paths=[_build.CSRC], with_cuda=True,
        extra_cflags=["-O2", "-std=c++17"],
        # found beside the module wherever the tree is copied to ($$ survives ninja, the
        # quotes survive the shell), and at the build-time path for the load check below
        extra_ldflags=[f"-L{_build.LIB_DIR}", "-lgpubridge_b200", "-Wl,-rpath,'$$ORIGIN'",
                       f"-Wl,-rpath,{_build.LIB_DIR}"],
        build_directory=WORK, verbose=verbose, is_python_module=False)
    os.replace(os.path.join(WORK, NAME + ".so"), OUT)
    with open(STAMP, "w") as fh:
        fh.write(_digest())
    return OUT


def load():
    """The extension module (built first when missing or stale)."""
    if NAME in sys.modules:
        return sys.modules[NAME]
    import torch  # noqa: F401 - libtorch must be loaded before the extension
    spec = importlib.util.spec_from_file_location(NAME, build())
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    sys.modules[NAME] = module
    return module


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv))
