"""The tcgen05 all-gather GEMM on one GPU (a team of one: the shard is the whole weight, and
the shard flag, the cross-proxy fence and the TMA / MMA / epilogue pipeline all run) against a
PyTorch fp32 reference."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("pair", [False, True], ids=["one-cta", "cta-pair"])
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 256), (1000, 1280, 200),
                                   (2048, 2048, 2048)])
def test_allgather_gemm_single_rank(M, N, K, pair):
    from gpubridge_b200.ops import fabric as F
    from gpubridge_b200.ops.gemm import AllGatherLinear
    device = torch.device("cuda", 0)
    team = F.create_single(device)
    try:
        torch.manual_seed(M + N + K)
        x = (torch.randn(M, K, device=device) * 0.5).to(torch.bfloat16)
        w = (torch.randn(N, K, device=device) * 0.5).to(torch.bfloat16)
        op = AllGatherLinear(team, N, K, pair=pair)
        for _ in range(2):                               # the second call reuses flags and buffers
            y = op(x, w)
        torch.cuda.synchronize(device)
        op.check()
        team.check()
        want = x.float() @ w.float().t()
        err = (y.float() - want).abs().max().item()
        assert err <= 2e-2 * want.abs().max().item() + 1e-2, err
    finally:
        team.close()


def _fused_on_a_team(rank, topology):
    """Every rank holds its rows of W; the fused kernel gathers the others' over NVLink while it
    already multiplies its own.  Checked against x @ W^T in fp32 with the whole weight, for both
    kernels, twice in a row (flags and staging are reused), then through ShardedLinear's
    autograd (input gradient and the averaged gradient of the own rows)."""
    import time
    from gpubridge_b200.ops.gemm import AllGatherLinear
    from gpubridge_b200.parallel.sharded_linear import ShardedLinear
    dev, world = topology.device, topology.world_size
    assert topology.fabric is not None
    timings = {}
    for pair in (False, True):
        for (M, N, K) in ((384, 512 * world, 256), (2048, 1024 * world, 1024)):
            g = torch.Generator().manual_seed(7)
            whole = (torch.randn(N, K, generator=g) * 0.5).to(torch.bfloat16)
            rows = N // world
            shard = whole[rank * rows:(rank + 1) * rows].to(dev).contiguous()
            x = (torch.randn(M, K, generator=torch.Generator().manual_seed(100 + rank)) * 0.5
                 ).to(torch.bfloat16).to(dev)
            op = AllGatherLinear(topology.fabric, N, K, pair=pair)
            for _ in range(2):
                y = op(x, shard)
            torch.cuda.synchronize(dev)
            op.check()
            topology.fabric.check()
            want = x.float().cpu() @ whole.float().t()
            err = (y.float().cpu() - want).abs().max().item()
            assert err <= 2e-2 * want.abs().max().item() + 1e-2, (pair, M, N, K, err)
            assert torch.equal(op.gathered.cpu(), whole), "the gathered weight must be the whole weight"
        # time the large shape: fused against all-gather (fabric) + cuBLAS
        big = torch.empty((N, K), dtype=torch.bfloat16, device=dev)
        import gpubridge_b200 as gb
        for label in ("fused", "gather+linear"):
            for _ in range(3):
                if label == "fused":
                    op(x, shard)
                else:
                    gb.all_gather_into_tensor(big, shard)
                    torch.nn.functional.linear(x, big)
            torch.cuda.synchronize(dev)
            gb.barrier()
            torch.cuda.synchronize(dev)
            t0 = time.perf_counter()
            for _ in range(10):
                if label == "fused":
                    op(x, shard)
                else:
                    gb.all_gather_into_tensor(big, shard)
                    torch.nn.functional.linear(x, big)
            torch.cuda.synchronize(dev)
            timings[f"{'pair' if pair else 'one'}/{label}"] = round((time.perf_counter() - t0) / 10 * 1e6, 1)
    layer = ShardedLinear(256, 512 * world, topology=topology)
    x = (torch.randn(64, 256, generator=torch.Generator().manual_seed(5 + rank)) * 0.5
         ).to(torch.bfloat16).to(dev).requires_grad_(True)
    y = layer(x)
    y.float().square().sum().backward()
    torch.cuda.synchronize(dev)
    slot = layer._slot()
    assert slot.op is not None, "the fused kernel must be the path under test"
    assert slot.gathers == 1, "a layer on its own reuses what forward left in the slot"
    whole = slot.buffer.float().cpu()
    xs = x.detach().float().cpu()
    assert torch.allclose(y.float().cpu(), xs @ whole.t(), atol=5e-2, rtol=2e-2)
    dy = (2 * y.detach().float()).to(torch.bfloat16).float().cpu()
    assert torch.allclose(x.grad.float().cpu(), dy @ whole, atol=0.5, rtol=5e-2)
    assert layer.weight.grad is not None and layer.weight.grad.shape == layer.weight.shape
    return timings


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2,
                    reason="needs at least two GPUs")
def test_allgather_gemm_on_a_team(tmp_path):
    from _harness import gpu_ranks, run_ranks
    out = run_ranks(gpu_ranks(2), _fused_on_a_team, tmp_path, timeout=240)
    print("2048 x 2048 x 1024 per call, us:", out[0])
