"""backend="gpubridge" in CPU simulation: DDP and FSDP2 bit for bit against a single process
on integer-valued float64 models, every collective, refusals, object collectives, subgroups,
HSDP on a (2, 2) mesh, point-to-point (reference: tests/test_torch_backend.py, test_p2p.py)."""
import pytest
import torch

from _harness import LAYOUTS, TWO_BY_TWO, run_ranks


def _integer_model(seed=0):
    torch.manual_seed(seed)
    model = torch.nn.Sequential(torch.nn.Linear(6, 8, dtype=torch.float64),
                                torch.nn.ReLU(),
                                torch.nn.Linear(8, 4, dtype=torch.float64))
    with torch.no_grad():
        for p in model.parameters():
            p.copy_(torch.randint(-3, 4, p.shape).double())
    return model


def _batch(rank):
    g = torch.Generator().manual_seed(50 + rank)
    return torch.randint(-2, 3, (4, 6), generator=g).double()


def _single_process_grads(world):
    model = _integer_model()
    x = torch.cat([_batch(r) for r in range(world)])
    model(x).sum().backward()
    return [p.grad / world for p in model.parameters()]


def _ddp(rank, world):
    import torch.distributed as dist
    from torch.nn.parallel import DistributedDataParallel as DDP
    model = DDP(_integer_model())
    model(_batch(rank)).sum().backward()
    for p, want in zip(model.parameters(), _single_process_grads(world)):
        assert torch.equal(p.grad, want)
    # every collective the backend carries
    t = torch.full((5,), float(rank))
    dist.all_reduce(t)
    assert torch.equal(t, torch.full((5,), float(sum(range(world)))))
    t = torch.full((3,), float(rank))
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    assert float(t[0]) == world - 1
    t = torch.full((3,), float(rank))
    dist.broadcast(t, src=2)
    assert float(t[0]) == 2
    out = torch.empty(world * 2)
    dist.all_gather_into_tensor(out, torch.full((2,), float(rank)))
    assert out.tolist() == [float(r) for r in range(world) for _ in range(2)]
    outs = [torch.empty(2) for _ in range(world)]
    dist.all_gather(outs, torch.full((2,), float(rank)))
    assert [float(o[0]) for o in outs] == [float(r) for r in range(world)]
    out = torch.empty(2)
    dist.reduce_scatter_tensor(out, torch.arange(world * 2.0))
    assert torch.equal(out, world * torch.arange(world * 2.0).view(world, 2)[rank])
    out = torch.empty(2)
    dist.reduce_scatter(out, [torch.full((2,), float(i)) for i in range(world)])
    assert float(out[0]) == world * rank
    dist.barrier()
    objs = [None] * world
    dist.all_gather_object(objs, {"rank": rank})
    assert [o["rank"] for o in objs] == list(range(world))
    gathered = [None] * world if rank == 0 else None
    dist.gather_object(rank * 10, gathered, dst=0)
    if rank == 0:
        assert gathered == [0, 10, 20, 30]
    with dist._coalescing_manager(device=torch.device("cpu"), async_ops=True) as cm:
        a, b = torch.ones(3) * rank, torch.ones(4) * rank
        dist.all_reduce(a)
        dist.all_reduce(b)
    cm.wait()
    assert float(a[0]) == sum(range(world)) and float(b[0]) == sum(range(world))
    # refusals happen before any communication
    for call in (lambda: dist.all_to_all_single(torch.empty(world), torch.empty(world)),
                 lambda: dist.reduce(torch.ones(2), dst=0)):
        with pytest.raises(NotImplementedError, match="doesn't support"):
            call()
    with pytest.raises(ValueError, match="PRODUCT"):
        dist.all_reduce(torch.ones(2), op=dist.ReduceOp.PRODUCT)
    return True


def test_ddp_and_every_collective(tmp_path):
    run_ranks(TWO_BY_TWO, _ddp, tmp_path, mode="backend")


def _fsdp(rank, world, hsdp):
    import torch.distributed as dist
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.fsdp import fully_shard
    import gpubridge_b200 as gb

    class Seen(gb.CollectiveObserver):
        def __init__(self):
            self.records = []

        def on_collective(self, record):
            self.records.append(record)

    model = _integer_model()
    if hsdp:
        mesh = init_device_mesh("cpu", (2, 2), mesh_dim_names=("replicate", "shard"))
    else:
        mesh = init_device_mesh("cpu", (world,))
    for layer in (model[0], model[2]):
        fully_shard(layer, mesh=mesh)
    fully_shard(model, mesh=mesh)
    dist.barrier()
    seen = Seen()
    gb.add_observer(seen)
    model(_batch(rank)).sum().backward()
    for p, want in zip(model.parameters(), _single_process_grads(world)):
        assert torch.equal(p.grad.full_tensor(), want), "FSDP2 gradient differs from one process"
    ops = [(r.op, r.policy, tuple(ph.name for ph in r.phases)) for r in seen.records]
    if hsdp:
        # shard groups are islands: native collectives with no bridge; replicate groups cross
        assert any(op == "all_gather_into_tensor" and policy == "native-only" for op, policy, _ in ops)
        assert any(op == "reduce_scatter_tensor" and policy == "native-only" for op, policy, _ in ops)
        bridged = [o for o in ops if o[0] == "all_reduce" and o[1] == "reduce-bridge-broadcast"]
        assert bridged and all("bridge" in phases for _, _, phases in bridged)
        assert not any("bridge" in phases for op, _, phases in ops if op != "all_reduce")
    return len(ops)


def test_fsdp2_matches_a_single_process(tmp_path):
    run_ranks(TWO_BY_TWO, _fsdp, tmp_path, False, mode="backend", timeout=180)


def test_hsdp_shard_groups_are_islands(tmp_path):
    run_ranks(TWO_BY_TWO, _fsdp, tmp_path, True, mode="backend", timeout=180)


def _p2p(rank, world):
    import torch.distributed as dist
    import gpubridge_b200 as gb
    dist.barrier()
    peer = (rank + 2) % world                       # the other island
    send = torch.full((1000,), float(rank))
    recv = torch.empty(1000)
    works = gb.batch_isend_irecv([dist.P2POp(dist.isend, send, peer, tag=3),
                                  dist.P2POp(dist.irecv, recv, peer, tag=3)])
    for w in works:
        w.wait()
    assert torch.equal(recv, torch.full((1000,), float(peer)))
    mate = rank ^ 1                                  # same island
    if rank < mate:
        dist.send(torch.full((7,), 5.0), dst=mate)
    else:
        got = torch.empty(7)
        dist.recv(got, src=mate)
        assert float(got[0]) == 5.0
    # a payload mismatch across islands raises instead of aborting the process
    dist.barrier()
    return True


def test_point_to_point_both_routes(tmp_path):
    run_ranks(TWO_BY_TWO, _p2p, tmp_path, mode="backend")


def _bad_setting(rank, world, path):
    import os
    from datetime import timedelta
    import torch.distributed as dist
    import gpubridge_b200  # noqa: F401
    if rank == 2:
        os.environ["GPUBRIDGE_POLICY"] = "fastest-one"
    dist.init_process_group("gpubridge", init_method=f"file://{path}", rank=rank, world_size=world,
                            timeout=timedelta(seconds=30))


def test_a_bad_setting_fails_every_rank(tmp_path):
    run_ranks(TWO_BY_TWO, _bad_setting, tmp_path, mode="raw",
              expect_error="unknown collective policy 'fastest-one'")
