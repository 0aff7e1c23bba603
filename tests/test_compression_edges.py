"""The codec oracle at its edges, in one process: values that are tiny, huge, subnormal or not
finite; the scale's exponent and its cap; payload sizes around block borders and zeroed padding;
the order and precision of the accumulation; what error feedback keeps, per buffer and part,
and that it stays bounded and finite step after step; several members quantising once each.
Every expectation is computed here from first principles, for both payload formats.
(Reference: tests/test_compression.py, the single-process half.)"""
import math

import pytest
import torch

from gpubridge_b200 import compression as C

FLT_MAX = torch.finfo(torch.float32).max


def roundtrip(mode, x, fmt="ref", residual=None, fill=0):
    n = x.numel()
    payload = torch.full((C.payload_nbytes(mode, n, fmt),), fill, dtype=torch.uint8)
    C.quantize_reference(mode, x, residual, payload, fmt)
    out = torch.empty(n)
    C.dequantize_accumulate_reference(mode, payload[None], out, fmt)
    return payload, out


# ---- what each mode applies to, and sizes -----------------------------------------------------------
def test_what_each_mode_compresses():
    floats = (torch.float16, torch.bfloat16, torch.float32, torch.float64)
    assert [C.applies("fp8", d) for d in floats] == [True] * 4
    assert [C.applies("bf16", d) for d in floats] == [False, False, True, True]      # 16-bit stays as it is
    for mode in C.MODES:
        assert not any(C.applies(mode, d) for d in (torch.int32, torch.int64, torch.uint8, torch.bool))
    assert not C.applies("", torch.float32) and not C.applies(None, torch.float32)
    with pytest.raises(ValueError, match="unknown bridge compression mode"):
        C.BridgeCompressor("fp4")
    with pytest.raises(ValueError, match="unknown codec format"):
        C.BridgeCompressor("fp8", "mx")
    with pytest.raises(ValueError, match="unknown compression mode"):
        C.quantize_reference("int8", torch.zeros(4), None, torch.zeros(16, dtype=torch.uint8))


@pytest.mark.parametrize("fmt, block", [("ref", 256), ("b200", 128)])
def test_payload_sizes_around_block_borders(fmt, block):
    for n in (1, 2, 3, 4, 5, block - 1, block, block + 1, 2 * block, 2 * block + 3, 70_001):
        blocks = math.ceil(n / block)
        assert C.n_blocks(n, fmt) == blocks
        assert C.payload_nbytes("fp8", n, fmt) == 4 * blocks + 4 * math.ceil(n / 4)
        assert C.payload_nbytes("bf16", n, fmt) == 4 * math.ceil(2 * n / 4)
        assert C.payload_nbytes("fp8", n, fmt) % 4 == 0 and C.payload_nbytes("bf16", n, fmt) % 4 == 0


@pytest.mark.parametrize("fmt", C.FORMATS)
@pytest.mark.parametrize("mode", C.MODES)
@pytest.mark.parametrize("n", [1, 3, 257, 130])
def test_padding_bytes_are_zeroed_whatever_was_there(mode, fmt, n):
    x = torch.randn(n)
    payload, _ = roundtrip(mode, x, fmt, fill=0xEE)
    used = 2 * n if mode == "bf16" else 4 * C.n_blocks(n, fmt) + n
    assert used <= payload.numel() < used + 4
    assert not payload[used:].any()
    again, _ = roundtrip(mode, x, fmt, fill=0x11)
    assert torch.equal(payload, again)                            # the payload is a function of the values alone


# ---- tiny, subnormal, non-finite, huge ---------------------------------------------------------------
@pytest.mark.parametrize("fmt", C.FORMATS)
@pytest.mark.parametrize("mode", C.MODES)
def test_a_block_of_only_tiny_values_sends_zeros(mode, fmt):
    x = torch.full((300,), 2.0 ** -101)
    x[::2] *= -1
    residual = torch.ones(300) * 2.0 ** -110
    payload, out = roundtrip(mode, x, fmt, residual)
    assert not out.any() and not residual.any()                    # flushed on the way in: nothing is owed either
    if mode == "fp8":
        nb = C.n_blocks(300, fmt)
        assert not payload[4 * nb:].any()
        assert torch.equal(payload[:4 * nb].view(torch.float32), torch.ones(nb))     # the scale of an empty block


@pytest.mark.parametrize("mode", C.MODES)
def test_a_block_of_float32_subnormals_sends_zeros_and_keeps_no_residual(mode):
    x = torch.full((256,), 1e-40)
    assert 0 < float(x[0]) < torch.finfo(torch.float32).tiny
    residual = torch.zeros(256)
    _, out = roundtrip(mode, x, "ref", residual)
    assert not out.any() and not residual.any()


@pytest.mark.parametrize("fmt", C.FORMATS)
@pytest.mark.parametrize("mode", C.MODES)
def test_non_finite_values_stay_non_finite_and_do_not_spoil_their_block(mode, fmt):
    torch.manual_seed(1)
    x = torch.randn(600)
    x[5], x[6], x[7] = float("inf"), float("-inf"), float("nan")
    residual = torch.zeros(600)
    _, out = roundtrip(mode, x, fmt, residual)
    assert not torch.isfinite(out[5:8]).any()
    if mode == "bf16":                                             # 16 bits keep which infinity it was
        assert out[5] == float("inf") and out[6] == float("-inf") and torch.isnan(out[7])
    rest = torch.ones(600, dtype=torch.bool)
    rest[5:8] = False
    assert torch.isfinite(out[rest]).all()
    clean = x.clone()
    clean[5:8] = 0                                                 # the block's scale ignores them
    assert ((out - x).abs()[rest] <= C.error_bound(mode, clean, fmt)[rest]).all()
    assert not residual[5:8].any() and torch.isfinite(residual).all()


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("mode", C.MODES)
def test_finite_values_near_float32s_max_arrive_finite_and_leave_finite_residuals(mode, dtype):
    x = torch.tensor([FLT_MAX, -FLT_MAX, FLT_MAX * 0.999, 3e38, 1.0, -2.5], dtype=dtype)
    if dtype == torch.float64:
        x = torch.cat([x, torch.tensor([1e300, -1e300], dtype=dtype)])      # beyond float32: saturates, stays finite
    residual = torch.zeros(x.numel())
    _, out = roundtrip(mode, x, "ref", residual)
    assert torch.isfinite(out).all() and torch.isfinite(residual).all()
    assert (out[:2].abs() >= 0.87 * FLT_MAX).all() and out[0] > 0 > out[1]
    if mode == "fp8":                                              # the capped scale's largest code, not infinity
        assert float(out[0]) == 448.0 * 2.0 ** 119 and float(residual[0]) == FLT_MAX - 448.0 * 2.0 ** 119


def test_the_fp8_scale_exponent_is_the_smallest_that_fits_and_is_capped():
    for k in (-20, -1, 0, 1, 7, 100):
        exact = torch.tensor([448.0 * 2.0 ** k])
        assert int(C.pow2_scale_exponent(exact)) == k              # amax / 2^k == 448 fits exactly
        above = torch.nextafter(exact, torch.tensor([float("inf")]))
        assert int(C.pow2_scale_exponent(above)) == k + 1
        below = torch.nextafter(exact, torch.tensor([0.0]))
        assert int(C.pow2_scale_exponent(below)) == k
    assert int(C.pow2_scale_exponent(torch.tensor([0.0]))) == 0
    assert int(C.pow2_scale_exponent(torch.tensor([FLT_MAX]))) == C.MAX_SCALE_EXP == 119
    assert 448.0 * 2.0 ** 119 <= FLT_MAX < 448.0 * 2.0 ** 120     # why 119: code * scale must fit float32
    one = torch.tensor([1.0])
    assert int(C.pow2_scale_exponent(one)) == -8 and 1.0 / 2.0 ** -8 <= 448 < 1.0 / 2.0 ** -9


def test_a_block_mixing_1e_4_and_3e38():
    x = torch.full((256,), 1e-4)
    x[0] = 3e38
    residual = torch.zeros(256)
    payload, out = roundtrip("fp8", x, "ref", residual)
    scale = float(payload[:4].view(torch.float32))
    assert scale == 2.0 ** 119
    assert abs(float(out[0]) - 3e38) <= 3e38 * 2 ** -4 and not out[1:].any()     # the small ones vanish on the wire
    assert torch.equal(residual[1:], x[1:])                                         # and are owed in full
    # they are never paid while that block keeps its giant: the debt stays what it is, finite
    for _ in range(5):
        _, out = roundtrip("fp8", x, "ref", residual)
    assert torch.isfinite(residual).all() and float(residual[1]) == pytest.approx(6e-4, rel=1e-5)


@pytest.mark.parametrize("fmt", C.FORMATS)
def test_the_b200_scale_is_amax_over_448_and_the_largest_value_is_exact(fmt):
    torch.manual_seed(2)
    x = torch.randn(128 * 3) * 7
    payload, out = roundtrip("fp8", x, fmt)
    size = C.block_size(fmt)
    for b in range(C.n_blocks(x.numel(), fmt)):
        block = x[b * size:(b + 1) * size]
        amax = float(block.abs().max())
        scale = float(payload[4 * b:4 * b + 4].view(torch.float32))
        if fmt == "b200":
            assert scale == float(torch.tensor(amax) / torch.tensor(448.0))
            where = int(block.abs().argmax())
            assert float(out[b * size + where]) == pytest.approx(float(block[where]), rel=1e-6)    # code 448 * amax / 448
        else:
            assert scale == 2.0 ** math.ceil(math.log2(amax / 448.0))


# ---- accumulation ------------------------------------------------------------------------------------
def test_dequantize_adds_members_in_order_in_float32():
    a, b, c = torch.tensor([2.0 ** 24]), torch.tensor([1.0]), torch.tensor([-2.0 ** 24])
    rows = []
    for v in (a, b, c):
        payload = torch.empty(C.payload_nbytes("bf16", 1), dtype=torch.uint8)
        C.quantize_reference("bf16", v, None, payload)
        rows.append(payload)
    out = torch.empty(1)
    C.dequantize_accumulate_reference("bf16", torch.stack(rows), out)
    assert float(out) == 0.0                                       # (2^24 + 1) + -2^24 in float32: the 1 is lost
    C.dequantize_accumulate_reference("bf16", torch.stack([rows[0], rows[2], rows[1]]), out)
    assert float(out) == 1.0                                       # (2^24 - 2^24) + 1: order is the rows' order
    wide = torch.empty(1, dtype=torch.float64)
    C.dequantize_accumulate_reference("bf16", torch.stack(rows), wide)
    assert float(wide) == 0.0                                      # still accumulated in float32, whatever comes out


def test_the_sum_is_rounded_once_to_the_output_type():
    torch.manual_seed(4)
    members = [torch.randn(1000) for _ in range(4)]
    rows = []
    for v in members:
        payload = torch.empty(C.payload_nbytes("fp8", 1000), dtype=torch.uint8)
        C.quantize_reference("fp8", v, None, payload)
        rows.append(payload)
    rows = torch.stack(rows)
    wide, narrow, half = torch.empty(1000), torch.empty(1000, dtype=torch.bfloat16), torch.empty(1000, dtype=torch.float16)
    for out in (wide, narrow, half):
        C.dequantize_accumulate_reference("fp8", rows, out)
    assert torch.equal(narrow, wide.to(torch.bfloat16)) and torch.equal(half, wide.to(torch.float16))
    scaled = torch.empty(1000)
    C.dequantize_accumulate_reference("fp8", rows, scaled, scale=4.0)
    assert torch.equal(scaled, wide / 4.0)                         # the fused average divides the float32 sum


def test_sums_that_cancel_to_almost_nothing_become_exact_zeros():
    v = torch.tensor([1.5, 2.0 ** -90])
    rows = []
    for sign in (1.0, -1.0):
        payload = torch.empty(C.payload_nbytes("bf16", 2), dtype=torch.uint8)
        C.quantize_reference("bf16", v * sign, None, payload)
        rows.append(payload)
    tail = torch.empty(C.payload_nbytes("bf16", 2), dtype=torch.uint8)
    C.quantize_reference("bf16", torch.tensor([0.0, 2.0 ** -101 * 1.5]), None, tail)
    out = torch.empty(2)
    C.dequantize_accumulate_reference("bf16", torch.stack(rows + [tail]), out)
    assert out.tolist() == [0.0, 0.0] and not torch.signbit(out).any()


@pytest.mark.parametrize("fmt", C.FORMATS)
@pytest.mark.parametrize("mode", C.MODES)
@pytest.mark.parametrize("members", [2, 4, 8])
def test_more_members_quantise_once_each_so_the_error_does_not_compound(members, mode, fmt):
    torch.manual_seed(members)
    values = [torch.randn(5000) * 3 for _ in range(members)]
    rows = []
    for v in values:
        payload = torch.empty(C.payload_nbytes(mode, 5000, fmt), dtype=torch.uint8)
        C.quantize_reference(mode, v, None, payload, fmt)
        rows.append(payload)
    out = torch.empty(5000)
    C.dequantize_accumulate_reference(mode, torch.stack(rows), out, fmt)
    exact = torch.stack(values).double().sum(0)
    allowed = sum(C.error_bound(mode, v, fmt).double() for v in values)
    slack = exact.abs() * members * 2.0 ** -23 + 1e-30             # the float32 additions themselves
    assert ((out.double() - exact).abs() <= allowed + slack).all()


# ---- error feedback ----------------------------------------------------------------------------------
@pytest.mark.parametrize("fmt", C.FORMATS)
@pytest.mark.parametrize("mode", C.MODES)
def test_error_feedback_keeps_the_accumulated_error_bounded(mode, fmt):
    """After T steps on one buffer, (sum of what was sent) differs from (sum of the inputs) by
    exactly the residual still owed - one quantisation's error, not T of them."""
    torch.manual_seed(9)
    residual = torch.zeros(4000)
    inputs, sent = torch.zeros(4000, dtype=torch.float64), torch.zeros(4000, dtype=torch.float64)
    for step in range(40):
        x = torch.randn(4000) * (1 + step % 3)
        before = residual.clone()
        _, out = roundtrip(mode, x, fmt, residual)
        inputs += x.double()
        sent += out.double()
        assert (residual.abs() <= C.error_bound(mode, x + before, fmt) * 1.0001).all()
    owed = (inputs - sent).float()
    assert torch.allclose(owed, residual, rtol=0, atol=float(inputs.abs().max()) * 2.0 ** -20)
    without = torch.zeros(4000, dtype=torch.float64)
    torch.manual_seed(9)
    for step in range(40):
        x = torch.randn(4000) * (1 + step % 3)
        _, out = roundtrip(mode, x, fmt)
        without += out.double()
    assert (inputs - sent).abs().mean() < (inputs - without).abs().mean()


@pytest.mark.parametrize("mode", C.MODES)
def test_error_feedback_stays_finite_step_after_step_at_float32s_max(mode):
    x = torch.tensor([FLT_MAX, -FLT_MAX, FLT_MAX / 3, 1.0] * 64)
    residual = torch.zeros(x.numel())
    for _ in range(50):
        _, out = roundtrip(mode, x, "ref", residual)
        assert torch.isfinite(out).all() and torch.isfinite(residual).all()


def test_a_compressor_keeps_one_residual_per_buffer_and_part():
    comp = C.BridgeCompressor("fp8")
    a, b = torch.randn(1000), torch.randn(1000)
    ra = comp.residual(C.buffer_key(a), a)
    assert ra.dtype == torch.float32 and ra.numel() == 1000 and not ra.any()
    assert comp.residual(C.buffer_key(a), a) is ra                 # the same buffer: the same debt
    assert comp.residual(C.buffer_key(b), b) is not ra
    first, second = a[:500], a[500:]
    r1, r2 = comp.residual(C.buffer_key(first, 0), first), comp.residual(C.buffer_key(second, 1), second)
    assert r1 is not r2 and r1.numel() == r2.numel() == 500
    assert C.buffer_key(first, 0) != C.buffer_key(first, 1)        # the same memory as another part is another debt
    # a buffer of another size at the same key starts afresh instead of adding a stale debt
    ra.fill_(1.0)
    shorter = a[:10]
    fresh = comp.residual(C.buffer_key(a), shorter)
    assert fresh.numel() == 10 and not fresh.any()
    comp.residual(C.buffer_key(b), b).fill_(3.0)
    other = C.BridgeCompressor("bf16")
    other.residual(C.buffer_key(b), b).fill_(5.0)
    comp.reset()
    assert not comp.residual(C.buffer_key(b), b).any()
    assert float(other.residual(C.buffer_key(b), b)[0]) == 5.0     # compressors do not share debts
    C.reset_error_feedback()
    assert not other.residual(C.buffer_key(b), b).any()


def test_a_compressors_rows_hold_its_own_payload_and_decompress_sums_them():
    torch.manual_seed(6)
    comps = [C.BridgeCompressor("fp8", "b200") for _ in range(3)]
    values = [torch.randn(777) for _ in range(3)]
    rows = [comp.compress(v, C.buffer_key(v), [10, 20, 30], me) for me, (comp, v) in enumerate(zip(comps, values))]
    assert all(r.shape == (3, C.payload_nbytes("fp8", 777, "b200")) and r.dtype == torch.uint8 for r in rows)
    gathered = torch.stack([rows[me][me] for me in range(3)])      # what the broadcasts of the bridge step do
    outs = []
    for comp in comps:
        out = torch.empty(777)
        comp.decompress(gathered, out)
        outs.append(out)
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[1], outs[2])          # every member: the same bits
    exact = torch.stack(values).sum(0)
    assert ((outs[0] - exact).abs() <= sum(C.error_bound("fp8", v, "b200") for v in values) + 1e-6).all()
    for comp, v in zip(comps, values):
        assert comp.residual(C.buffer_key(v), v).any()             # each keeps what its payload left out


def test_bound_helpers_are_tight_enough_to_mean_something():
    torch.manual_seed(8)
    x = torch.randn(100_000)
    for mode, fmt in (("bf16", "ref"), ("fp8", "ref"), ("fp8", "b200")):
        _, out = roundtrip(mode, x, fmt)
        err, bound = (out - x).abs(), C.error_bound(mode, x, fmt)
        assert (err <= bound).all()
        assert float((err / bound).max()) > 0.4                    # somewhere the bound is nearly reached
        assert float(bound.mean()) < (0.005 if mode == "bf16" else 0.08)
