"""The checked build of the native library (``-DGB_BOUNDS``): it compiles for sm_100a, exports a
range table per kernel file, and the table round-trips; on GPUs it runs the collectives with
every access compared against the memory the host allowed (``tests/test_gpu_bounds.py``)."""
import ctypes
import os
import subprocess
import sys

import pytest

from gpubridge_b200.ops import _build, _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.skipif(not os.path.exists(_build.LIB_BOUNDS), reason="the checked library is not built")
def test_checked_library_exports_a_table_per_kernel_file():
    lib = ctypes.CDLL(_build.LIB_BOUNDS)
    for unit in _lib.BOUNDS_UNITS:
        assert hasattr(lib, f"gb_bounds_set_{unit}") and hasattr(lib, f"gb_bounds_get_{unit}")
    plain = ctypes.CDLL(_build.LIB)
    assert not hasattr(plain, "gb_bounds_set_collectives")


def test_table_layout_matches_the_header():
    text = open(os.path.join(ROOT, "gpubridge_b200", "csrc", "gb_common.cuh")).read()
    assert f"#define GB_BOUNDS_RANGES {_lib.BOUNDS_RANGES}" in text
    assert ctypes.sizeof(_lib.GbBoundsTable) == 16 * _lib.BOUNDS_RANGES + 8 + 32 + 8


def test_the_variable_selects_the_library():
    code = "from gpubridge_b200.ops import _lib; print(_lib.path())"
    env = dict(os.environ, GPUBRIDGE_BOUNDS="1")
    out = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, cwd=ROOT)
    assert out.stdout.strip().endswith("libgpubridge_b200_bounds.so"), out.stderr
