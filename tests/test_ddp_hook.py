"""``DistributedDataParallel`` with ``ddp_comm_hook`` on a job joined through ``init``: DDP keeps
its buckets and its overlap, every bucket is averaged through the chosen policy.  Gradients are
checked exactly (integer data), over layouts and policies, with several buckets, a compressed bridge, and a bucket whose collective fails.
(Reference: tests/test_ddp.py.)"""
import pytest
import torch

from _harness import LAYOUTS, run_ranks


def _net(dtype=torch.float64):
    torch.manual_seed(0)
    net = torch.nn.Sequential(torch.nn.Linear(16, 32), torch.nn.ReLU(), torch.nn.Linear(32, 32), torch.nn.ReLU(),
                              torch.nn.Linear(32, 4)).to(dtype)
    with torch.no_grad():
        for p in net.parameters():
            p.copy_(torch.randint(-2, 3, p.shape).to(dtype))
    return net


def _batch(rank, dtype=torch.float64):
    generator = torch.Generator().manual_seed(100 + rank)
    return torch.randint(-3, 4, (8, 16), generator=generator).to(dtype)


def _expected(world, dtype=torch.float64):
    """The average over the ranks' local gradients, computed in one process."""
    total = None
    for r in range(world):
        net = _net(dtype)
        net(_batch(r, dtype)).sum().backward()
        grads = [p.grad.clone() for p in net.parameters()]
        total = grads if total is None else [a + b for a, b in zip(total, grads)]
    return [g / world for g in total]


def _train(rank, topology, cap_mb):
    from torch.nn.parallel import DistributedDataParallel as DDP
    import gpubridge_b200 as gb

    class Count(gb.CollectiveObserver):
        def __init__(self):
            self.buckets = []

        def on_collective(self, record):
            self.buckets.append((record.op, record.reduce_op, record.nbytes))

    counter = Count()
    gb.add_observer(counter)
    net = _net()
    model = DDP(net, bucket_cap_mb=cap_mb)
    model.register_comm_hook(None, gb.ddp_comm_hook)
    for _ in range(2):                                             # the second step uses DDP's rebuilt buckets
        model.zero_grad(set_to_none=True)
        model(_batch(rank)).sum().backward()
    want = _expected(topology.world_size)
    assert all(torch.equal(p.grad, w) for p, w in zip(net.parameters(), want))
    buckets = [b for b in counter.buckets if b[0] == "all_reduce"]
    assert buckets and all(op == "avg" for _, op, _ in buckets)
    return len(buckets), sum(n for _, _, n in buckets)


@pytest.mark.parametrize("layout, policy", [
    ("2+2", "auto"), ("interleaved", "pipelined-reduce-bridge-broadcast"), ("3+1", "sharded-bridge"),
    ("2+2", "sharded-bridge"), ("3+1", "flat-gloo"), ("single-vendor", "auto")])
def test_ddp_with_the_hook_averages_gradients_exactly(tmp_path, layout, policy):
    out = run_ranks(LAYOUTS[layout], _train, tmp_path, 25, init={"policy": policy}, timeout=120)
    parameter_bytes = sum(p.numel() for p in _net().parameters()) * 8
    assert all(total == 2 * parameter_bytes for _, total in out)   # every gradient went through once per step


def test_small_buckets_mean_several_collectives_per_step(tmp_path):
    out = run_ranks(LAYOUTS["2+2"], _train, tmp_path, 0.004, timeout=120)
    assert all(count > 2 for count, _ in out), out                 # more than one bucket per step
    assert len({count for count, _ in out}) == 1


def _compressed(rank, topology):
    from torch.nn.parallel import DistributedDataParallel as DDP
    import gpubridge_b200 as gb
    net = _net(torch.float32)
    model = DDP(net)
    model.register_comm_hook(None, gb.ddp_comm_hook)
    model(_batch(rank, torch.float32)).sum().backward()
    want = _expected(topology.world_size, torch.float32)
    worst = max(float((p.grad - w).abs().max() / (w.abs().max() + 1e-9)) for p, w in zip(net.parameters(), want))
    flat = torch.cat([p.grad.reshape(-1) for p in net.parameters()])
    return worst, flat.numpy().tobytes()                           # bytes travel between processes as they are


def test_a_compressed_bridge_keeps_every_rank_on_the_same_gradients(tmp_path):
    out = run_ranks(LAYOUTS["2+2"], _compressed, tmp_path, env={"GPUBRIDGE_BRIDGE_COMPRESSION": "fp8"}, timeout=120)
    assert all(0 < worst < 0.1 for worst, _ in out)                # lossy, within fp8's bound
    assert all(flat == out[0][1] for _, flat in out)    # but the same bits everywhere


def _failing_bucket(rank, topology):
    from torch.nn.parallel import DistributedDataParallel as DDP
    import gpubridge_b200 as gb
    net = _net()
    model = DDP(net)
    model.register_comm_hook(None, gb.ddp_comm_hook)
    model(_batch(rank)).sum().backward()                           # a good step first
    original = type(topology.policy).all_reduce

    def broken(self, tensor, topology_, op="sum", **kwargs):
        raise OSError("the link went down")

    type(topology.policy).all_reduce = broken
    try:
        model.zero_grad(set_to_none=True)
        with pytest.raises((RuntimeError, OSError), match="link went down"):
            model(_batch(rank)).sum().backward()
    finally:
        type(topology.policy).all_reduce = original
    with pytest.raises(RuntimeError):                              # and the rank stays poisoned: no silent carrying on
        gb.all_reduce(torch.ones(4))
    return True


def test_a_failed_bucket_makes_backward_raise_on_every_rank(tmp_path):
    assert run_ranks(LAYOUTS["2+2"], _failing_bucket, tmp_path, timeout=120) == [True] * 4
