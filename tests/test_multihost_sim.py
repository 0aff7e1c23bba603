"""Several hosts without a cluster: every rank names its host through GPUBRIDGE_SIM_HOSTNAME;
``GPUBRIDGE_SPLIT_TEST=node`` turns every second host into another island, and the collectives
run over the composed (host-bridged) path, as a job that spans boxes would."""
import torch

from _harness import expected_sum, rank_tensor, run_ranks


def _two_hosts(rank, world, path):
    import os
    import warnings
    from datetime import timedelta
    os.environ["GPUBRIDGE_SIM_HOSTNAME"] = f"box{rank // 2}"
    os.environ["GPUBRIDGE_SPLIT_TEST"] = "node"
    import gpubridge_b200 as gb
    with warnings.catch_warnings():
        warnings.simplefilter("ignore", gb.SplitTestWarning)
        topology = gb.init(f"file://{path}", rank=rank, world_size=world, timeout=timedelta(seconds=40))
    try:
        islands = [list(i.ranks) for i in topology.layout.islands]
        assert islands == [[0, 1], [2, 3]], islands
        assert topology.split_test == "node" and topology.fabric is None
        assert {p.hostname for p in topology.peers} == {"box0", "box1"}
        for n in (5, 70_001):
            t = rank_tensor(rank, n)
            gb.all_reduce(t)
            assert torch.equal(t, expected_sum(world, n))
        out = torch.empty(world * 3)
        gb.all_gather_into_tensor(out, torch.full((3,), float(rank)))
        assert out.tolist() == [float(r) for r in range(world) for _ in range(3)]
        return topology.policy_name
    finally:
        gb.destroy()


def test_islands_by_host(tmp_path):
    out = run_ranks(("nvidia",) * 4, _two_hosts, tmp_path, mode="raw")
    assert set(out) == {"reduce-bridge-broadcast"}
