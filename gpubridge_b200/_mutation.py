"""Test-only switches that undo one stream-ordering step each, so the GPU tests that guard
those steps can be shown to fail without them (``python -m gpubridge_b200.kit.stream_mutations``).
Nothing sets ``GPUBRIDGE_TEST_MUTATION`` outside that program.

    comm-ignores-caller    a synchronous fused collective starts without waiting for the work
                           queued on the caller's stream
    caller-ignores-comm    ... and the caller's stream does not wait for it afterwards
    async-ignores-caller   an asynchronous fused collective starts without that wait
    wait-skips-stream      Work.wait() returns without ordering the caller's stream
    staging-ignores-caller the pinned staging copies start without waiting for the caller's stream
"""
from __future__ import annotations

import os

NAMES = ("comm-ignores-caller", "caller-ignores-comm", "async-ignores-caller",
         "wait-skips-stream", "staging-ignores-caller")


def mutated(name: str) -> bool:
    return os.environ.get("GPUBRIDGE_TEST_MUTATION", "") == name
