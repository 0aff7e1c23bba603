"""The data-parallel trainer's optimizer inside backward (a bucket is updated as soon as its
gradients are in) against the same optimizer called once after backward: same arithmetic, so
the same bits, on one CPU process; the step count advances once per step either way."""
import copy

import torch
import torch.nn as nn

from gpubridge_b200.parallel.trainer import DataParallelTrainer


def _model():
    torch.manual_seed(3)
    return nn.Sequential(nn.Linear(24, 40), nn.GELU(), nn.Linear(40, 40), nn.GELU(),
                         nn.LayerNorm(40), nn.Linear(40, 8))


def _loss(model, x, y):
    return nn.functional.mse_loss(model(x), y)


def test_updates_inside_backward_equal_one_update_after_it():
    first = _model()
    second = copy.deepcopy(first)
    inside = DataParallelTrainer(first, _loss, autocast=None, bucket_mb=0.002,
                                 optimizer_in_backward=True, lr=1e-2)
    after = DataParallelTrainer(second, _loss, autocast=None, bucket_mb=0.002,
                                optimizer_in_backward=False, lr=1e-2)
    assert len(inside._buckets) >= 3
    g = torch.Generator().manual_seed(0)
    for _ in range(4):
        x, y = torch.randn(16, 24, generator=g), torch.randn(16, 8, generator=g)
        a, b = inside.step(x, y), after.step(x, y)
        assert torch.equal(a, b)
        assert torch.equal(inside.flat_param, after.flat_param)
        assert torch.equal(inside.optimizer.m, after.optimizer.m)
        assert torch.equal(inside.optimizer.v, after.optimizer.v)
        assert float(inside.flat_grad.abs().max()) == 0.0
    assert float(inside.optimizer.state[2]) == float(after.optimizer.state[2]) == 4.0


def test_accumulated_micro_batches_update_once():
    first = _model()
    second = copy.deepcopy(first)
    inside = DataParallelTrainer(first, _loss, autocast=None, bucket_mb=0.002,
                                 optimizer_in_backward=True)
    after = DataParallelTrainer(second, _loss, autocast=None, bucket_mb=0.002,
                                optimizer_in_backward=False)
    g = torch.Generator().manual_seed(1)
    micro = [(torch.randn(8, 24, generator=g), torch.randn(8, 8, generator=g)) for _ in range(3)]
    inside.step_accumulated(micro)
    after.step_accumulated(micro)
    assert torch.equal(inside.flat_param, after.flat_param)
    assert float(inside.optimizer.state[2]) == 1.0
