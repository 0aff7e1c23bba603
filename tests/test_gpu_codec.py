"""The sm_100a codec kernels against the PyTorch oracle, bit for bit (the reference tests
its Triton kernels the same way: tests/test_compression_kernels.py)."""
import pytest
import torch

from gpubridge_b200 import compression as C

pytestmark = pytest.mark.gpu

SIZES = (1, 7, 255, 256, 257, 4099, 1_000_003)


def _values(n, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(n, generator=g) * torch.exp(torch.randn(n, generator=g) * 6)
    if n > 16:
        x[3], x[5], x[7], x[8], x[9] = float("inf"), float("nan"), 0.0, -0.0, 1e-35
        x[11], x[12] = 3.3e38, -3.4e38
    return x.to(dtype)


def _bits(t):
    view = {2: torch.int16, 4: torch.int32, 8: torch.int64}[t.element_size()]
    return t.contiguous().view(view)


@pytest.mark.parametrize("fmt", C.FORMATS)
@pytest.mark.parametrize("mode", C.MODES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16, torch.float64])
def test_quantize_matches_oracle(mode, dtype, fmt):
    if dtype not in C.APPLIES_TO[mode]:
        pytest.skip("mode does not apply to this dtype")
    from gpubridge_b200.ops import codec
    for n in SIZES:
        for with_residual in (False, True):
            x = _values(n, dtype, n)
            res_cpu = torch.randn(n) * 1e-3 if with_residual else None
            res_gpu = res_cpu.cuda() if with_residual else None
            want = torch.empty(C.payload_nbytes(mode, n, fmt), dtype=torch.uint8)
            C.quantize_reference(mode, x, res_cpu, want, fmt)
            got = torch.full_like(want, 0xAB).cuda()
            codec.quantize(mode, x.cuda(), res_gpu, got, fmt)
            torch.cuda.synchronize()
            assert torch.equal(got.cpu(), want), (n, with_residual)
            if with_residual:
                assert torch.equal(_bits(res_gpu.cpu()), _bits(res_cpu)), (n, "residual")


@pytest.mark.parametrize("fmt", C.FORMATS)
@pytest.mark.parametrize("mode", C.MODES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16, torch.float64])
def test_dequantize_matches_oracle(mode, dtype, fmt):
    if dtype not in C.APPLIES_TO[mode]:
        pytest.skip("mode does not apply to this dtype")
    from gpubridge_b200.ops import codec
    for n in SIZES:
        for members in (1, 2, 3):
            rows = torch.empty((members, C.payload_nbytes(mode, n, fmt)), dtype=torch.uint8)
            for m in range(members):
                x = _values(n, torch.float32, 100 * n + m)
                if m:                      # row 0 keeps its NaN and infinities
                    x[~torch.isfinite(x)] = 1.0
                C.quantize_reference(mode, x, None, rows[m], fmt)
            want = torch.empty(n, dtype=dtype)
            C.dequantize_accumulate_reference(mode, rows, want, fmt)
            got = torch.empty(n, dtype=dtype, device="cuda")
            codec.dequantize_accumulate(mode, rows.cuda(), got, fmt)
            torch.cuda.synchronize()
            a, b = _bits(got.cpu()), _bits(want)
            nan = torch.isnan(want)
            assert torch.equal(a[~nan], b[~nan]), (n, members)
            assert torch.isnan(got.cpu()[nan]).all()


def test_error_bounds_hold_on_device():
    from gpubridge_b200.ops import codec
    n = 1 << 20
    x = torch.randn(n) * torch.exp(torch.randn(n) * 3)
    for mode in C.MODES:
        for fmt in C.FORMATS:
            payload = torch.empty(C.payload_nbytes(mode, n, fmt), dtype=torch.uint8, device="cuda")
            codec.quantize(mode, x.cuda(), None, payload, fmt)
            out = torch.empty(n, device="cuda")
            codec.dequantize_accumulate(mode, payload[None], out, fmt)
            err = (out.cpu() - x).abs()
            assert (err <= C.error_bound(mode, x, fmt) * (1 + 1e-6)).all(), (mode, fmt)
