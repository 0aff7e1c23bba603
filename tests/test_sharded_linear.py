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
    # the weight gradient in pieces (a batched GEMM and an asynchronous reduce-scatter per piece)
    pieced = ShardedLinear(16, 24, topology=topology, dtype=torch.float64)
    pieced.grad_chunks = 3 if rows % 3 == 0 else 2
    x2 = xs[rank].clone().requires_grad_(True)
    pieced(x2).square().sum().backward()
    assert torch.allclose(pieced.weight.grad, want, atol=1e-10)
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


def _stack(rank, topology):
    """Three equal layers share one slot: correct gradients, one whole weight resident, and a
    second gather in backward for every layer but the last."""
    from gpubridge_b200.parallel import sharded_linear as sl
    world = topology.world_size
    rows = 16 // world
    counts = {}
    for reshard in (True, False):
        sl.release_slots()
        layers = [sl.ShardedLinear(16, 16, topology=topology, dtype=torch.float64, seed=s,
                                   reshard_after_forward=reshard) for s in range(3)]
        x0 = torch.randn(4, 16, generator=torch.Generator().manual_seed(20 + rank)).double()
        x = x0.clone().requires_grad_(True)
        h = x
        for layer in layers:
            h = torch.tanh(layer(h))
        h.sum().backward()
        slots = {id(layer._slot()): layer._slot() for layer in layers}
        counts[reshard] = (len(slots), sum(s.gathers for s in slots.values()))
        # oracle on whole weights: every rank's loss, weight gradients averaged over ranks
        wholes = [_whole_weight(16, 16, seed=s).double() for s in range(3)]
        grads = [[] for _ in wholes]
        for r in range(world):
            ws = [w.clone().requires_grad_(True) for w in wholes]
            xr = torch.randn(4, 16, generator=torch.Generator().manual_seed(20 + r)).double().requires_grad_(True)
            hr = xr
            for w in ws:
                hr = torch.tanh(hr @ w.t())
            hr.sum().backward()
            for i, w in enumerate(ws):
                grads[i].append(w.grad)
            if r == rank:
                assert torch.allclose(x.grad, xr.grad, atol=1e-10), reshard
        for i, layer in enumerate(layers):
            want = torch.stack(grads[i]).mean(0)[rank * rows:(rank + 1) * rows]
            assert torch.allclose(layer.weight.grad, want, atol=1e-10), (reshard, i)
    sl.release_slots()
    return counts


def test_equal_layers_share_one_gathered_weight(tmp_path):
    counts = run_ranks(LAYOUTS["2+2"], _stack, tmp_path)[0]
    assert counts[True] == (1, 5)         # one slot; 3 forward gathers + 2 in backward
    assert counts[False] == (3, 3)        # a slot per layer; nothing gathered twice
