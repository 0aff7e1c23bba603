"""The arithmetic of the bench tools, in this process: message sizes, bus-bandwidth factors,
how a sweep turns into a thresholds file, the sweep matrix's reading of result files, the
point-to-point bench's routes and data pattern, and the timing loop on a pretend topology
(slowest rank per trial, median over trials, the time limit agreed between ranks).
(Reference: the helper cases of tests/test_gpu_kit.py and tests/test_bench_p2p.py.)"""
import json
import types

import pytest
import torch

from gpubridge_b200 import policies, topology
from gpubridge_b200.bench import bench_all_reduce, bench_matrix, bench_p2p


def test_sizes_double_from_the_smallest_to_the_largest():
    assert bench_all_reduce.sizes(4096, 65536) == [4096, 8192, 16384, 32768, 65536]
    assert bench_all_reduce.sizes(1000, 5000) == [1000, 2000, 4000]
    assert bench_all_reduce.sizes(8, 8) == [8] and bench_all_reduce.sizes(16, 8) == []
    assert len(bench_all_reduce.sizes(4 << 10, 1 << 30)) == 19     # 4 KiB .. 1 GiB: the sweep of record


def test_bus_bandwidth_factors_follow_the_usual_definitions():
    factors = bench_all_reduce.BUS
    for n in (2, 4, 8):
        assert factors["all_reduce"](n) == pytest.approx(2 * (n - 1) / n)
        assert factors["all_gather"](n) == factors["reduce_scatter"](n) == pytest.approx((n - 1) / n)
        assert factors["broadcast"](n) == 1.0
    # 1 GiB all-reduced over 8 ranks in 2.6 ms: 1.75 bytes on the bus per byte of payload
    assert (1 << 30) / 2.6e-3 * factors["all_reduce"](8) / 1e9 == pytest.approx(722.7, rel=0.01)


def rows(*entries):
    return [{"op": "all_reduce", "target": target, "bytes": size, "ms": ms} for target, size, ms in entries]


def test_the_fastest_policy_per_size_becomes_a_rule_and_neighbours_merge(tmp_path):
    path = tmp_path / "t.json"
    measured = rows(("policy:flat-gloo", 4096, 0.1), ("policy:reduce-bridge-broadcast", 4096, 0.3),
                    ("policy:flat-gloo", 8192, 0.2), ("policy:reduce-bridge-broadcast", 8192, 0.3),
                    ("policy:flat-gloo", 16384, 0.9), ("policy:reduce-bridge-broadcast", 16384, 0.4),
                    ("policy:flat-gloo", 32768, 2.0), ("policy:sharded-bridge", 32768, 0.5),
                    ("ours", 4096, 0.001), ("nccl", 8192, 0.001))            # not policies: never rules
    measured.append({"op": "broadcast", "target": "policy:flat-gloo", "bytes": 32768, "ms": 0.0001})
    bench_all_reduce.write_thresholds(measured, str(path))
    saved = json.loads(path.read_text())
    assert saved["rules"] == [{"max_bytes": 8192, "policy": "flat-gloo"},
                              {"max_bytes": 16384, "policy": "reduce-bridge-broadcast"},
                              {"max_bytes": None, "policy": "sharded-bridge"}]
    loaded = policies.load_thresholds(str(path), 1 << 20)          # and the policy can read it back
    assert loaded["rules"] == saved["rules"]
    bench_all_reduce.write_thresholds(rows(("ours", 4096, 0.1)), str(path))   # nothing to choose from
    assert json.loads(path.read_text())["rules"] == [{"max_bytes": None, "policy": "auto"}]


def test_the_matrix_reads_both_shapes_of_result_files(tmp_path):
    listed = tmp_path / "a.json"
    listed.write_text(json.dumps(rows(("ours", 4096, 0.1), ("nccl", 4096, 0.2)) +
                                 [{"op": "broadcast", "target": "ours", "bytes": 4096, "ms": 9}]))
    wrapped = tmp_path / "b.json"
    wrapped.write_text(json.dumps({"rows": [{"target": "ours", "bytes": "8192", "ms": 0.3}]}))       # no op: all_reduce
    assert bench_matrix.load(listed) == {"ours": {4096: rows(("ours", 4096, 0.1))[0]}, "nccl": {4096: rows(("nccl", 4096, 0.2))[0]}}
    assert list(bench_matrix.load(wrapped)["ours"]) == [8192]
    assert [bench_matrix.human(n) for n in (512, 4096, 1 << 20, 3 << 30, 1536)] == ["512", "4K", "1M", "3G", "1536"]
    assert [bench_p2p.human(n) for n in (1 << 10, 5 << 20)] == ["1K", "5M"]
    assert [r[0] for r in bench_matrix.RANGES] == ["under 256 KB", "256 KB to under 64 MB", "64 MB and up"]
    assert bench_matrix.RANGES[0][2] == bench_matrix.RANGES[1][1] and bench_matrix.RANGES[1][2] == bench_matrix.RANGES[2][1]


def test_the_point_to_point_bench_picks_one_peer_per_route():
    def fake(vendors):
        return types.SimpleNamespace(layout=topology.plan_topology(vendors))
    assert bench_p2p.routes(fake(["nvidia", "nvidia", "amd", "amd"])) == {"bridge": 2, "native": 1}
    assert bench_p2p.routes(fake(["nvidia", "amd", "nvidia", "amd"])) == {"bridge": 1, "native": 2}
    assert bench_p2p.routes(fake(["nvidia", "amd"])) == {"bridge": 1}                 # an island of one has no native peer
    assert bench_p2p.routes(fake(["amd", "amd", "amd"])) == {"native": 1}


def test_the_data_pattern_is_exact_distinct_and_built_in_pieces():
    small = bench_p2p.pattern(1000, torch.device("cpu"))
    assert small.dtype == torch.float32 and torch.equal(small, (torch.arange(1000) % 251).float())
    large = bench_p2p.pattern((1 << 20) + 5, torch.device("cpu"))                    # crosses a piece border
    assert torch.equal(large, (torch.arange((1 << 20) + 5) % 251).float())
    assert bench_p2p.pattern(0, torch.device("cpu")).numel() == 0


class World:
    """A world group of one process that plays every rank's part: ``all_reduce`` combines this
    rank's value with what the other ranks are said to have measured."""

    def __init__(self, others):
        self.others, self.calls = list(others), 0

    def barrier(self):
        pass

    def all_reduce(self, tensor, op):
        self.calls += 1
        if tensor.dtype == torch.float64 and op == "max":          # a trial's time: the slowest rank counts
            other = self.others.pop(0) if self.others else 0.0
            tensor.fill_(max(float(tensor), other))


def test_a_trial_counts_the_slowest_rank_and_the_median_is_reported():
    world = World([5.0, 50.0, 7.0, 6.0, 8.0])
    pretend = types.SimpleNamespace(device=torch.device("cpu"), world_group=world)
    calls = []
    ms = bench_all_reduce.time_calls(lambda: calls.append(1), pretend, trials=5, seconds=60, warmup=2)
    assert ms == 7.0                                               # median of the other ranks' (slower) times
    assert len(calls) == 2 + 5                                     # warm-up, then one call per trial
    calls.clear()
    bench_all_reduce.time_calls(lambda: calls.append(1), types.SimpleNamespace(
        device=torch.device("cpu"), world_group=World([])), trials=3, seconds=60, warmup=0, inner=4)
    assert len(calls) == 12                                        # inner back-to-back calls per trial


def test_the_time_limit_ends_the_trials_on_every_rank_together():
    import time

    class Slow(World):
        def all_reduce(self, tensor, op):
            super().all_reduce(tensor, op)
            if tensor.dtype == torch.float32:                      # the "are we over time" vote
                tensor.fill_(1.0 if self.calls >= 4 else float(tensor))     # another rank says stop after 2 trials

    pretend = types.SimpleNamespace(device=torch.device("cpu"), world_group=Slow([]))
    calls = []
    bench_all_reduce.time_calls(lambda: calls.append(1), pretend, trials=50, seconds=3600, warmup=0)
    assert len(calls) == 2                                         # stopped because SOME rank was over time
    started = time.monotonic()
    bench_all_reduce.time_calls(lambda: time.sleep(0.05), types.SimpleNamespace(
        device=torch.device("cpu"), world_group=World([])), trials=1000, seconds=0.2, warmup=0)
    assert time.monotonic() - started < 2
