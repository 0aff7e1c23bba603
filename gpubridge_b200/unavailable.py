"""Transports whose system libraries are not present in this build.

The reference ships a UCX bridge (C++ over libucp) that refuses to load with a clear message
when the library or its headers are missing (reference: src/gpubridge/ucx/__init__.py:45-46).
``ucp/api/ucp.h`` does not exist in this image, and on one NVSwitch box the bridge is NVLink, so
the name stays known and says why it can't be used.  (The verbs bridge's endpoint is built and
tested over an in-process fabric: :mod:`gpubridge_b200.rdma`.)
"""
from __future__ import annotations

import ctypes.util

_NEEDS = {"ucx": ("ucp", "libucp (UCX)")}


def load(name: str) -> None:
    lib, label = _NEEDS[name]
    found = ctypes.util.find_library(lib)
    raise ImportError(
        f"{label} {'was found but its headers are not part of this build' if found else 'is not installed'}; "
        "use bridge='nvlink' on one NVSwitch box, or 'multitcp' / 'gloo' across nodes")
