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


# ---- the profiler leaves no trace and counts what is really kept ---------------------------------------
def test_a_layer_that_raises_leaves_everything_as_it_was():
    class Breaks(nn.Module):
        def forward(self, x):
            raise RuntimeError("this layer cannot run")

    layers = [nn.Linear(8, 8), Breaks(), nn.Linear(8, 8)]
    before = [p.detach().clone() for layer in layers for p in layer.parameters()]
    example = torch.randn(2, 8)
    state = torch.random.get_rng_state()
    with pytest.raises(RuntimeError, match="cannot run"):
        balance.profile_layers(layers, example, torch.device("cpu"), trials=1)
    assert torch.equal(state, torch.random.get_rng_state())
    for layer in layers:
        assert all(p.device.type == "cpu" and p.grad is None for p in layer.parameters())
    assert all(torch.equal(a, b) for a, b in zip(before, (p for layer in layers for p in layer.parameters())))


def test_shared_parameters_stay_shared_and_are_counted_where_they_are_used():
    shared = nn.Linear(8, 8)

    class Twice(nn.Module):
        def __init__(self, inner):
            super().__init__()
            self.inner = inner

        def forward(self, x):
            return self.inner(self.inner(x))

    layers = [Twice(shared), Twice(shared)]
    costs = balance.profile_layers(layers, torch.randn(4, 8), torch.device("cpu"), trials=1)
    assert layers[0].inner is layers[1].inner is shared            # profiling worked on copies
    assert costs[0].state_bytes == costs[1].state_bytes == (64 + 8) * 16
    # the middle activation is saved once although two matmuls read it; the weights are not activations
    assert 4 * 8 * 4 <= costs[0].activation_bytes <= 3 * 4 * 8 * 4


def test_a_layer_without_parameters_and_an_integer_input_are_profiled():
    table = nn.Embedding(50, 16)
    layers = [table, nn.ReLU(), nn.Flatten()]
    tokens = torch.randint(0, 50, (4, 7))
    costs = balance.profile_layers(layers, tokens, torch.device("cpu"), trials=1, warmup=0)
    assert [c.out_bytes for c in costs] == [4 * 7 * 16 * 4] * 3
    assert costs[0].state_bytes == 50 * 16 * 16 and costs[1].state_bytes == costs[2].state_bytes == 0
    assert costs[1].activation_bytes >= 4 * 7 * 16 * 4             # ReLU keeps its output for backward
    other = balance.profile_layers(layers, tokens, torch.device("cpu"), trials=1, state_bytes_per_parameter=4)
    assert other[0].state_bytes == 50 * 16 * 4


def test_a_sparse_inputs_whole_storage_counts():
    dense = torch.zeros(6, 10)
    dense[0, 1], dense[3, 4], dense[5, 9] = 1.0, 2.0, 3.0
    sparse = dense.to_sparse()
    pieces = balance._storages(sparse)
    assert len(pieces) == 2 and sum(size for _, size in pieces) == 2 * 3 * 8 + 3 * 4       # indices + values
    csr = dense.to_sparse_csr()
    assert len(balance._storages(csr)) == 3
    assert balance._storages(dense) == [(dense.untyped_storage().data_ptr(), 6 * 10 * 4)]
    view = dense[2:4]
    assert balance._storages(view) == balance._storages(dense)     # a view keeps the whole storage alive


def test_a_slower_second_device_gets_fewer_layers_and_the_expected_speedup():
    layers = 24
    fast, slow = [1.0] * layers, [3.0] * layers
    even = max(balance.evaluate([12, 12], [fast, slow], [0.0] * (layers - 1), [1e12]))
    plan = balance.partition([fast, slow], [0.0] * (layers - 1), [1e12])
    assert plan.split == [18, 6] and plan.bottleneck_ms == pytest.approx(18.0)
    assert even / plan.bottleneck_ms == pytest.approx(2.0)         # 36 ms -> 18 ms per microbatch
    # a slow link between the stages moves the cut to where less crosses it
    boundary = [1e6] * (layers - 1)
    boundary[15] = 1e3
    near = balance.partition([fast, slow], boundary, [1e5])
    assert near.split == [16, 8]


def test_bad_input_is_refused():
    with pytest.raises(ValueError):
        balance.partition([], [], [])
    with pytest.raises(ValueError):
        balance.partition([[1.0, 1.0], [1.0]], [1.0], [1.0])       # stages disagree on the layer count
    with pytest.raises(ValueError):
        balance.partition([[1.0] * 3] * 4, [1.0] * 2, [1.0] * 3)   # more stages than layers
    with pytest.raises(ValueError):
        balance.partition([[1.0] * 4] * 2, [1.0] * 2, [1.0])       # boundaries: one per cut position
    with pytest.raises(ValueError):
        balance.partition([[1.0] * 4] * 2, [1.0] * 3, [1.0, 1.0])  # links: one per neighbouring pair
    with pytest.raises(ValueError):
        balance.in_flight("1f1b", 0, 4)
