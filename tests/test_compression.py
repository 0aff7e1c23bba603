"""The codec against torch's float8 type and its documented error bounds, error feedback,
and compressed bridge steps of every bridged policy in CPU simulation (reference:
tests/test_compression.py)."""
import pytest
import torch

from _harness import LAYOUTS, run_ranks
from gpubridge_b200 import compression as C


def test_e4m3_codes_match_torch_float8():
    codes = torch.arange(256, dtype=torch.int32).to(torch.uint8)
    values = C.e4m3_decode(codes)
    want = codes.view(torch.float8_e4m3fn).float()
    finite = torch.isfinite(want)
    assert torch.equal(values[finite], want[finite])
    assert torch.isnan(values[0x7F]) and torch.isnan(values[0xFF])
    x = torch.randn(200_000) * torch.exp(torch.randn(200_000) * 2)
    x = x.clamp(-448, 448)
    got = C.e4m3_encode(x)
    ref = x.to(torch.float8_e4m3fn).view(torch.uint8)
    ref = torch.where(x == 0, torch.zeros_like(ref), ref)
    assert torch.equal(got, ref)
    assert int(C.e4m3_encode(torch.tensor([1000.0]))) == 0x7E          # saturates at 448
    assert int(C.e4m3_encode(torch.tensor([-0.0]))) == 0


@pytest.mark.parametrize("fmt", C.FORMATS)
@pytest.mark.parametrize("mode", C.MODES)
def test_error_bounds(mode, fmt):
    torch.manual_seed(3)
    for n in (1, 255, 256, 257, 70_001):
        x = torch.randn(n) * torch.exp(torch.randn(n) * 4)
        payload = torch.empty(C.payload_nbytes(mode, n, fmt), dtype=torch.uint8)
        residual = torch.zeros(n)
        C.quantize_reference(mode, x, residual, payload, fmt)
        out = torch.empty(n)
        C.dequantize_accumulate_reference(mode, payload[None], out, fmt)
        err = (out - x).abs()
        assert (err <= C.error_bound(mode, x, fmt)).all()
        assert torch.equal(residual, x - out)                           # what was left out


def test_payload_layout_and_special_values():
    n = 300
    x = torch.randn(n)
    x[0], x[1], x[2] = float("inf"), float("nan"), 1e-35
    payload = torch.full((C.payload_nbytes("fp8", n),), 0xAB, dtype=torch.uint8)
    residual = torch.zeros(n)
    C.quantize_reference("fp8", x, residual, payload)
    assert C.payload_nbytes("fp8", n) == 4 * 2 + 300
    scales = payload[:8].view(torch.float32)
    assert all(float(s) == 2.0 ** round(torch.log2(s).item()) for s in scales)   # powers of two
    assert payload[8] == 0x7F and payload[9] == 0x7F and payload[10] == 0       # inf, nan, tiny
    assert residual[0] == 0 and residual[1] == 0
    assert C.payload_nbytes("bf16", 3) == 8 and C.payload_nbytes("fp8", 5, "b200") == 4 + 8


def test_error_feedback_beats_no_feedback():
    torch.manual_seed(0)
    n, steps = 4096, 200
    grads = [torch.randn(n) * 0.01 for _ in range(steps)]
    truth = sum(g.double() for g in grads)
    for mode in C.MODES:
        with_ef, without = torch.zeros(n, dtype=torch.float64), torch.zeros(n, dtype=torch.float64)
        residual = torch.zeros(n)
        payload = torch.empty(C.payload_nbytes(mode, n), dtype=torch.uint8)
        out = torch.empty(n)
        for g in grads:
            C.quantize_reference(mode, g, residual, payload)
            C.dequantize_accumulate_reference(mode, payload[None], out)
            with_ef += out.double()
            C.quantize_reference(mode, g, None, payload)
            C.dequantize_accumulate_reference(mode, payload[None], out)
            without += out.double()
        assert (with_ef - truth).abs().mean() * 5 < (without - truth).abs().mean()


def _compressed(rank, topology, mode, fmt):
    import gpubridge_b200 as gb
    world, islands = topology.world_size, topology.layout.islands
    for dtype in (torch.float32, torch.bfloat16):
        if dtype not in C.APPLIES_TO[mode]:
            continue
        for n in (1024, 5000):
            values = [torch.randn(n, generator=torch.Generator().manual_seed(1234 + r)).to(dtype)
                      for r in range(world)]
            exact = sum(v.double() for v in values)
            t = values[rank].clone()
            gb.all_reduce(t)
            # every rank ends with identical bits
            gathered = torch.empty(world * n, dtype=dtype)
            gb.all_gather_into_tensor(gathered, t)
            assert all(torch.equal(row, gathered.view(world, n)[0]) for row in gathered.view(world, n))
            # the documented bound: one quantisation per island, plus rounding
            bound = torch.zeros(n)
            for island in islands:
                part = sum(values[r].float() for r in island.ranks)
                bound += C.error_bound(mode, part, fmt)
            slack = 2.0 ** -7 * exact.abs().float() + 1e-5 if dtype is torch.bfloat16 else 1e-5
            assert ((t.double() - exact).abs().float() <= bound * 1.01 + slack + 0.02 *
                    (dtype is torch.bfloat16)).all(), (mode, dtype, n)
    # integer dtypes and MAX are never compressed
    t = torch.full((10,), rank, dtype=torch.int64)
    gb.all_reduce(t)
    assert torch.equal(t, torch.full((10,), sum(range(world)), dtype=torch.int64))
    gb.reset_error_feedback()
    return True


@pytest.mark.parametrize("policy", ["reduce-bridge-broadcast", "pipelined-reduce-bridge-broadcast",
                                    "sharded-bridge"])
@pytest.mark.parametrize("mode,fmt", [("fp8", "ref"), ("bf16", "ref"), ("fp8", "b200")])
def test_compressed_bridge(tmp_path, policy, mode, fmt):
    run_ranks(LAYOUTS["2+2"], _compressed, tmp_path, mode, fmt, init={"policy": policy},
              env={"GPUBRIDGE_BRIDGE_COMPRESSION": mode, "GPUBRIDGE_CODEC_FORMAT": fmt,
                   "GPUBRIDGE_CHUNK_BYTES": "512"})


def test_ranks_must_agree_on_compression(tmp_path):
    run_ranks(LAYOUTS["2+2"], _disagree, tmp_path, mode="raw",
              expect_error="disagree on GPUBRIDGE_BRIDGE_COMPRESSION")


def _disagree(rank, world, path):
    import os
    from datetime import timedelta
    import gpubridge_b200 as gb
    if rank == 1:
        os.environ["GPUBRIDGE_BRIDGE_COMPRESSION"] = "fp8"
    gb.init(f"file://{path}", rank=rank, world_size=world, timeout=timedelta(seconds=30))
