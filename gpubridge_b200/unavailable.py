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


def info() -> dict:
    """What is known about each unavailable transport (``python -m gpubridge_b200.unavailable info``)."""
    import os
    out = {}
    for name, (lib, label) in _NEEDS.items():
        out[name] = {"needs": label, "library_found": ctypes.util.find_library(lib) is not None,
                     "header_found": os.path.exists("/usr/include/ucp/api/ucp.h")}
    return out


def main(argv: list[str]) -> int:
    import json
    import sys
    command = argv[0] if argv else "info"
    if command == "info":
        print(json.dumps(info()))
        return 0
    if command == "build":
        try:
            load("ucx")
        except ImportError as failure:
            print(f"nothing to build: {failure}", file=sys.stderr)
            return 1
    print("usage: python -m gpubridge_b200.unavailable [build|info]", file=sys.stderr)
    return 2


if __name__ == "__main__":
    import sys
    sys.exit(main(sys.argv[1:]))
