"""pytest configuration: the ``gpu`` marker, and a clean environment for every test."""
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
             "GPUBRIDGE_ALGO", "GPUBRIDGE_ASYNC_QUEUE")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA GPU (run with pytest -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
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
