"""The fused GEMM + reduce-scatter (csrc/gb_gemm_rs.cu) on hardware, against a plain PyTorch
fp32 reference of the same operation: on one GPU (a team of one: the epilogue stores into the
own workspace, the tail adds one slot) and on a team of two (rows cross NVLink).

The kernel has not run on hardware yet: the tests join the suite with GPUBRIDGE_TEST_GEMM_RS=1
until it has."""
import os

import pytest
import torch

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(os.environ.get("GPUBRIDGE_TEST_GEMM_RS") != "1",
                                 reason="joins the suite with GPUBRIDGE_TEST_GEMM_RS=1")]

SHAPES = [(256, 512, 128), (384, 264, 72), (2048, 1024, 512), (640, 2048, 4096)]     # P, Q, R


def _inputs(rank, P, Q, R, dev):
    g = torch.Generator().manual_seed(40 + rank)
    a = (torch.randn(P, R, generator=g) * 0.5).to(torch.bfloat16)
    b = (torch.randn(Q, R, generator=g) * 0.5).to(torch.bfloat16)
    return a.to(dev), b.to(dev)


def _reference(world, rank, P, Q, R):
    """What a bf16 reduce-scatter of fp32-accumulated products gives: every rank's product
    rounded to bf16, the roundings added in fp32 in rank order, divided, this rank's rows."""
    total = torch.zeros(P, Q)
    for r in range(world):
        a, b = _inputs(r, P, Q, R, "cpu")
        total += (a.float() @ b.float().t()).to(torch.bfloat16).float()
    rows = P // world
    return (total / world)[rank * rows:(rank + 1) * rows]


def test_one_rank(monkeypatch):
    # a first run: keep every device-side wait short, so that a mistake ends in seconds
    monkeypatch.setenv("GPUBRIDGE_WAIT_TIMEOUT_MS", "5000")
    from gpubridge_b200.ops import fabric as fabric_mod
    from gpubridge_b200.ops.gemm import GemmReduceScatter
    dev = torch.device("cuda", 0)
    fabric = fabric_mod.create_single(dev)
    try:
        op = GemmReduceScatter(fabric)
        for P, Q, R in SHAPES:
            a, b = _inputs(0, P, Q, R, dev)
            want = _reference(1, 0, P, Q, R)
            for dtype in (torch.bfloat16, torch.float32):
                for _ in range(2):                        # twice: both halves of the region
                    out = op(a, b, divide=1, out_dtype=dtype)
                torch.cuda.synchronize(dev)
                op.check()
                tol = 2e-2 if dtype is torch.bfloat16 else 1e-2
                assert torch.allclose(out.float().cpu(), want, atol=tol * (R ** 0.5) * 0.25, rtol=tol), (P, Q, R, dtype)
    finally:
        torch.cuda.synchronize(dev)
        fabric.close()


def _on_a_team(rank, topology):
    from gpubridge_b200.ops.gemm import GemmReduceScatter
    from gpubridge_b200.parallel.sharded_linear import ShardedLinear
    dev, world = topology.device, topology.world_size
    op = GemmReduceScatter(topology.fabric)
    for P, Q, R in SHAPES:
        a, b = _inputs(rank, P, Q, R, dev)
        want = _reference(world, rank, P, Q, R)
        for _ in range(3):
            out = op(a, b, divide=world, out_dtype=torch.float32)
        torch.cuda.synchronize(dev)
        op.check()
        assert torch.allclose(out.cpu(), want, atol=5e-3 * (R ** 0.5), rtol=1e-2), (P, Q, R)
    # through the layer: the fused gradient against the two-kernel path
    os.environ["GPUBRIDGE_GEMM_RS"] = "1"
    fused = ShardedLinear(256, 512 * world, topology=topology)
    os.environ["GPUBRIDGE_GEMM_RS"] = "0"
    plain = ShardedLinear(256, 512 * world, topology=topology)
    x = (torch.randn(128, 256, generator=torch.Generator().manual_seed(7 + rank)) * 0.5).to(torch.bfloat16).to(dev)
    for layer in (fused, plain):
        layer(x.clone().requires_grad_(True)).float().square().sum().backward()
    torch.cuda.synchronize(dev)
    assert fused._slot().scatter is not None, "the fused kernel must be the path under test"
    assert torch.allclose(fused.weight.grad.float(), plain.weight.grad.float(), atol=0.5, rtol=5e-2)
    return True


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2,
                    reason="needs at least two GPUs")
def test_on_a_team_of_two(tmp_path):
    from _harness import gpu_ranks, run_ranks
    run_ranks(gpu_ranks(2), _on_a_team, tmp_path, timeout=240,
              env={"GPUBRIDGE_WAIT_TIMEOUT_MS": "10000", "NCCL_NVLS_ENABLE": "0", "GPUBRIDGE_NVLS": "0"})
