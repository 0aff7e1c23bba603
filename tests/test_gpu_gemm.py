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
