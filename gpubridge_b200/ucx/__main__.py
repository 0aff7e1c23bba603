"""``python -m gpubridge_b200.ucx build | info``: compile the UCX worker ahead of a job, or say
what is known about UCX on this machine."""
from __future__ import annotations

import json
import sys

from gpubridge_b200 import ucx


def main(argv: list[str]) -> int:
    command = argv[0] if argv else "info"
    if command == "info":
        print(json.dumps(ucx.info()))
        return 0
    if command == "build":
        try:
            print(ucx.build(force="--force" in argv[1:]))
            return 0
        except ucx.Unavailable as why:
            print(f"nothing built: {why}", file=sys.stderr)
            return 1
    print("usage: python -m gpubridge_b200.ucx [build [--force] | info]", file=sys.stderr)
    return 2


if __name__ == "__main__":
    sys.exit(main(sys.argv[1:]))
