"""The stage partitioner against brute force, memory limits, and layer profiling on CPU
(reference: tests/test_balance.py)."""
import itertools
import random

import pytest
import torch
from torch import nn

from gpubridge_b200 import balance


def _brute(layer_ms, boundary, bw):
    stages, layers = len(layer_ms), len(layer_ms[0])
    best = None
    for cuts in itertools.combinations(range(1, layers), stages - 1):
        split = [b - a for a, b in zip((0, *cuts), (*cuts, layers))]
        worst = max(balance.evaluate(split, layer_ms, boundary, bw))
        if best is None or worst < best - 1e-12:
            best = worst
    return best


def test_partition_is_optimal():
    rng = random.Random(7)
    for _ in range(60):
        stages, layers = rng.randint(1, 4), rng.randint(4, 9)
        layer_ms = [[rng.uniform(0.5, 5.0) * (1 + s) for _ in range(layers)] for s in range(stages)]
        boundary = [rng.uniform(1e5, 5e6) for _ in range(layers - 1)]
        bw = [rng.uniform(5e5, 5e6) for _ in range(stages - 1)]
        plan = balance.partition(layer_ms, boundary, bw)
        assert sum(plan.split) == layers and min(plan.split) >= 1
        assert plan.bottleneck_ms == pytest.approx(_brute(layer_ms, boundary, bw))
        assert plan.stage_ms == balance.evaluate(plan.split, layer_ms, boundary, bw)


def test_faster_device_gets_more_layers_and_memory_limits_bind():
    layer_ms = [[1.0] * 12, [2.0] * 12]
    plan = balance.partition(layer_ms, [1000.0] * 11, [1e9])
    assert plan.split == [8, 4]
    limited = balance.partition(layer_ms, [1000.0] * 11, [1e9], state_bytes=[10] * 12,
                                activation_bytes=[5] * 12,
                                in_flight=balance.in_flight("1f1b", 2, 4), memory_bytes=[100, None])
    assert limited.split == [5, 7]          # 5 * (10 + 2 * 5) = 100 fits, 6 does not
    with pytest.raises(ValueError, match="no split fits"):
        balance.partition(layer_ms, [1000.0] * 11, [1e9], state_bytes=[10] * 12,
                          activation_bytes=[5] * 12, in_flight=[4, 4], memory_bytes=[10, 10])
    with pytest.raises(ValueError):
        balance.partition(layer_ms, [1.0] * 11, [1e9], memory_bytes=[1, 1])
    assert balance.in_flight("gpipe", 3, 8) == [8, 8, 8]
    assert balance.in_flight("1f1b", 3, 8) == [3, 2, 1]
    with pytest.raises(ValueError):
        balance.in_flight("zigzag", 2, 2)
    with pytest.raises(ValueError):
        balance.evaluate([3, 3], layer_ms, [1.0] * 11, [1e9])


def test_profile_layers_leaves_the_model_alone():
    torch.manual_seed(0)
    layers = [nn.Linear(16, 32), nn.Sequential(nn.Tanh(), nn.Dropout(0.5)), nn.Linear(32, 4)]
    before = [p.detach().clone() for layer in layers for p in layer.parameters()]
    example = torch.randn(8, 16)
    state = torch.random.get_rng_state()
    costs = balance.profile_layers(layers, example, torch.device("cpu"), trials=2)
    assert torch.equal(state, torch.random.get_rng_state())
    assert [c.out_bytes for c in costs] == [8 * 32 * 4, 8 * 32 * 4, 8 * 4 * 4]
    assert costs[0].state_bytes == (16 * 32 + 32) * 16 and costs[1].state_bytes == 0
    assert all(c.ms >= 0 and c.activation_bytes >= 0 for c in costs)
    assert costs[0].activation_bytes >= 8 * 16 * 4          # the input is saved for backward
    after = [p for layer in layers for p in layer.parameters()]
    assert all(torch.equal(a, b) and b.grad is None for a, b in zip(before, after))
