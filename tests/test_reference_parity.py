"""Bit-compatibility with the reference's own codec and wire formats, checked against the
reference package itself when it is installed under ``baseline/_ref`` (its pure-Python codec
runs on CPU).  Skipped when it is not there."""
import importlib
import os
import sys

import pytest
import torch

from gpubridge_b200 import compression as mine

REF = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "baseline", "_ref")


@pytest.fixture(scope="module")
def ref():
    if not os.path.isdir(os.path.join(REF, "gpubridge")):
        pytest.skip("the reference is not installed under baseline/_ref")
    sys.path.insert(0, REF)
    try:
        yield importlib.import_module("gpubridge.compression")
    finally:
        sys.path.remove(REF)


def _bits(t):
    return t.contiguous().view({2: torch.int16, 4: torch.int32, 8: torch.int64}[t.element_size()])


def test_payloads_and_residuals_are_bit_identical(ref):
    torch.manual_seed(0)
    for n in (1, 7, 255, 256, 257, 4099, 100_003):
        for dtype in (torch.float32, torch.bfloat16, torch.float16, torch.float64):
            for mode in ("bf16", "fp8"):
                if dtype not in ref.APPLIES_TO[mode]:
                    continue
                x = (torch.randn(n) * torch.exp(torch.randn(n) * 8)).to(dtype)
                if n > 10:
                    x[3], x[5], x[7], x[8], x[9] = float("inf"), float("nan"), 0.0, -0.0, 1e-35
                r1 = torch.randn(n) * 1e-3
                r2 = r1.clone()
                p1 = torch.empty(ref.payload_nbytes(mode, n), dtype=torch.uint8)
                p2 = torch.empty(mine.payload_nbytes(mode, n), dtype=torch.uint8)
                ref.quantize_reference(mode, x, r1, p1)
                mine.quantize_reference(mode, x, r2, p2)
                assert torch.equal(p1, p2), (n, dtype, mode)
                assert torch.equal(_bits(r1), _bits(r2)), (n, dtype, mode)
                rows = torch.stack([p1, p1, p2])
                o1, o2 = torch.empty(n, dtype=dtype), torch.empty(n, dtype=dtype)
                ref.dequantize_accumulate_reference(mode, rows, o1)
                mine.dequantize_accumulate_reference(mode, rows, o2)
                assert torch.equal(_bits(o1), _bits(o2)), (n, dtype, mode)


def test_constants_and_layout_match(ref):
    assert (mine.BLOCK, mine.FP8_MAX, mine.MAX_SCALE_EXP, mine.TINY) == \
        (ref.BLOCK, ref.FP8_MAX, ref.MAX_SCALE_EXP, ref.TINY)
    assert mine.APPLIES_TO == ref.APPLIES_TO
    for n in (0, 1, 255, 256, 1000):
        for mode in ("bf16", "fp8"):
            assert mine.payload_nbytes(mode, n) == ref.payload_nbytes(mode, n)


def test_public_names_cover_the_reference(ref):
    import gpubridge
    import gpubridge_b200
    missing = [name for name in gpubridge.__all__ if not hasattr(gpubridge_b200, name)]
    assert missing == []
    import gpubridge.topology as rt
    from gpubridge_b200 import topology as mt
    ours = set(mt.PeerInfo.__dataclass_fields__)
    assert set(rt.PeerInfo.__dataclass_fields__) <= ours
