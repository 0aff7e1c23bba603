"""Transports whose system libraries are not present in this build.

The reference ships a UCX bridge (C++ over libucp) and an ibverbs bridge (Rust over
libibverbs); both refuse to load with a clear message when the library or its headers
are missing (reference: src/gpubridge/ucx/__init__.py:45-46, verbs/__init__.py:63-64).
Neither ``ucp/api/ucp.h`` nor ``infiniband/verbs.h`` exists in this image, and on one
NVSwitch box the bridge is NVLink, so the names stay known and say why they can't be used.
"""
from __future__ import annotations

import ctypes.util

_NEEDS = {"ucx": ("ucp", "libucp (UCX)"), "verbs": ("ibverbs", "libibverbs")}


def load(name: str) -> None:
    lib, label = _NEEDS[name]
    found = ctypes.util.find_library(lib)
    raise ImportError(
        f"{label} {'was found but its headers are not part of this build' if found else 'is not installed'}; "
        "use bridge='nvlink' on one NVSwitch box, or 'multitcp' / 'gloo' across nodes")
