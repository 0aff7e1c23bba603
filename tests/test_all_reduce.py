"""Every policy on every layout gives the exact sum (integer-valued data), identical to the
flat-gloo oracle (the reference's method: tests/test_all_reduce.py:19-41)."""
import pytest
import torch

from _harness import LAYOUTS, expected_sum, rank_tensor, run_ranks

SIZES = (1, 17, 4099)
BRIDGED = ("reduce-bridge-broadcast", "pipelined-reduce-bridge-broadcast", "sharded-bridge")


def _all_reduce(rank, topology, policy_name):
    import gpubridge_b200 as gb
    assert topology.policy_name == policy_name or policy_name == "auto"
    for dtype in (torch.float32, torch.bfloat16, torch.int64):
        for n in SIZES:
            t = rank_tensor(rank, n, dtype)
            gb.all_reduce(t)
            assert torch.equal(t, expected_sum(topology.world_size, n, dtype)), (dtype, n)
    t = rank_tensor(rank, 33)
    gb.all_reduce(t, gb.ReduceOp.AVG)
    assert torch.allclose(t, expected_sum(topology.world_size, 33) / topology.world_size)
    for op, fold in ((gb.ReduceOp.MAX, torch.maximum), (gb.ReduceOp.MIN, torch.minimum)):
        t = rank_tensor(rank, 9)
        gb.all_reduce(t, op)
        want = rank_tensor(0, 9)
        for r in range(1, topology.world_size):
            want = fold(want, rank_tensor(r, 9))
        assert torch.equal(t, want)
    return topology.policy_name


@pytest.mark.parametrize("layout", ["2+2", "interleaved", "3+1", "1+3"])
@pytest.mark.parametrize("policy", ["auto", *BRIDGED, "flat-gloo", "auto-tuned"])
def test_bridged_layouts(tmp_path, layout, policy):
    names = run_ranks(LAYOUTS[layout], _all_reduce, tmp_path, policy, init={"policy": policy},
                      env={"GPUBRIDGE_CHUNK_BYTES": "64"})
    assert len(set(names)) == 1
    if policy == "auto":
        assert names[0] == "reduce-bridge-broadcast"


@pytest.mark.parametrize("layout", ["single-vendor", "single-rank"])
@pytest.mark.parametrize("policy", ["auto", "native-only", "flat-gloo"])
def test_single_island(tmp_path, layout, policy):
    names = run_ranks(LAYOUTS[layout], _all_reduce, tmp_path, policy, init={"policy": policy})
    if policy == "auto":
        assert names[0] == "native-only"


def test_policy_that_does_not_fit_fails_everywhere(tmp_path):
    run_ranks(LAYOUTS["single-vendor"], _all_reduce, tmp_path, "sharded-bridge",
              init={"policy": "sharded-bridge"}, expect_error="doesn't apply to this cluster")
