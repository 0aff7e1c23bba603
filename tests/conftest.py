"""pytest configuration: the ``gpu`` marker, a clean environment for every test, and shards
(``GPUBRIDGE_TEST_SHARD=K/N`` keeps every N-th test file, starting with the K-th, so that a
CI matrix of N jobs runs the suite once between them)."""
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for path in (ROOT, os.path.dirname(os.path.abspath(__file__))):
    if path not in sys.path:
        sys.path.insert(0, path)

_SETTINGS = ("GPUBRIDGE_BRIDGE_COMPRESSION", "GPUBRIDGE_PINNED_STAGING", "GPUBRIDGE_POLICY",
             "GPUBRIDGE_BRIDGE", "GPUBRIDGE_THRESHOLDS", "GPUBRIDGE_CHUNK_BYTES",
             "GPUBRIDGE_SPLIT_TEST", "GPUBRIDGE_ISLANDS", "GPUBRIDGE_VENDOR",
             "GPUBRIDGE_CPU_ONLY", "GPUBRIDGE_CODEC_FORMAT", "GPUBRIDGE_FABRIC",
             "GPUBRIDGE_ALGO", "GPUBRIDGE_ASYNC_QUEUE", "GPUBRIDGE_P2P_CHUNK_BYTES",
             "GPUBRIDGE_UCX_CHUNK_BYTES", "GPUBRIDGE_UCX_DIRECT_MIN_BYTES", "GPUBRIDGE_JOB_ID")
#: every setting of the host-staged bridges (a shell that exports one must not change what a test means)
_SETTING_PREFIXES = ("GPUBRIDGE_VERBS_", "GPUBRIDGE_MULTITCP_")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA GPU (run with pytest -m gpu on a B200)")


def shard_of(files: list[str], spec: str) -> set[str]:
    """The files of shard ``K/N`` (K from 1): round-robin over the sorted names, so shards
    stay balanced as files are added."""
    k, n = (int(v) for v in spec.split("/"))
    if not 1 <= k <= n:
        raise ValueError(f"GPUBRIDGE_TEST_SHARD={spec}: want K/N with 1 <= K <= N")
    return {f for i, f in enumerate(sorted(set(files))) if i % n == k - 1}


def pytest_collection_modifyitems(config, items):
    spec = os.environ.get("GPUBRIDGE_TEST_SHARD", "").strip()
    if spec:
        keep = shard_of([str(item.fspath) for item in items], spec)
        dropped = [item for item in items if str(item.fspath) not in keep]
        items[:] = [item for item in items if str(item.fspath) in keep]
        config.hook.pytest_deselected(items=dropped)
    import torch
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA GPU on this machine")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(autouse=True)
def _clean_settings(monkeypatch):
    """Bit-exact tests must not inherit compression or policy settings from the shell."""
    for name in _SETTINGS:
        monkeypatch.delenv(name, raising=False)
    for name in [n for n in os.environ if n.startswith(_SETTING_PREFIXES)]:
        monkeypatch.delenv(name, raising=False)
