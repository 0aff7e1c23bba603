"""ShardedLinear against a plain Linear holding the whole weight: forward, input gradient and
the averaged, row-sharded weight gradient (CPU ranks through the composed collectives; the
fused tcgen05 path has its own GPU test)."""
import math

import pytest
import torch

from _harness import LAYOUTS, run_ranks


def _whole_weight(out_features, in_features, seed=0):
    g = torch.Generator().manual_seed(seed)
    return torch.empty(out_features, in_features).uniform_(-1, 1, generator=g) / math.sqrt(in_features)


def _layer(rank, topology):
    from gpubridge_b200.parallel.sharded_linear import ShardedLinear
    world = topology.world_size
    layer = ShardedLinear(16, 24, topology=topology, dtype=torch.float64)
    whole = _whole_weight(24, 16).double()
    rows = 24 // world
    assert torch.equal(layer.weight.detach(), whole[rank * rows:(rank + 1) * rows])
    xs = [torch.randn(5, 3, 16, generator=torch.Generator().manual_seed(10 + r)).double()
          for r in range(world)]
    x = xs[rank].clone().requires_grad_(True)
    y = layer(x)
    assert torch.allclose(y, xs[rank] @ whole.t(), atol=1e-12)
    y.square().sum().backward()
    # oracle: every rank's loss on the whole weight, gradients averaged over ranks
    grads, dx = [], None
    for r in range(world):
        w = whole.clone().requires_grad_(True)
        xr = xs[r].clone().requires_grad_(True)
        (xr @ w.t()).square().sum().backward()
        grads.append(w.grad)
        if r == rank:
            dx = xr.grad
    want = torch.stack(grads).mean(0)[rank * rows:(rank + 1) * rows]
    assert torch.allclose(layer.weight.grad, want, atol=1e-10)
    assert torch.allclose(x.grad, dx, atol=1e-10)
    return True


@pytest.mark.parametrize("layout", ["2+2", "single-vendor"])
def test_matches_a_whole_linear(tmp_path, layout):
    run_ranks(LAYOUTS[layout], _layer, tmp_path)


def test_single_process():
    from gpubridge_b200.parallel.sharded_linear import ShardedLinear
    layer = ShardedLinear(8, 12, dtype=torch.float32)
    x = torch.randn(4, 8, requires_grad=True)
    y = layer(x)
    assert torch.allclose(y, x @ _whole_weight(12, 8).t(), atol=1e-6)
    y.sum().backward()
    assert layer.weight.grad.shape == (12, 8) and x.grad.shape == (4, 8)
