"""The native path of the C++ front end on hardware.

One GPU: a team of one (the same kernels, no peers) behind a ``GbBackend`` whose stand-in
Python group only hands out the engine - every collective must take the native path, be
ordered with the caller's stream both ways, and leave a Work and a future that behave like
torch's own.  Two or more GPUs: ``backend="gpubridge_native"`` end to end (exact sums on
integer-valued data, all_gather / reduce_scatter / broadcast, DDP)."""
import os

import pytest
import torch

from _harness import expected_sum, gpu_ranks, rank_tensor, run_ranks

pytestmark = pytest.mark.gpu
NGPU = torch.cuda.device_count() if torch.cuda.is_available() else 0


class _OneRankGroup:
    """What GbBackend asks of its Python group, for a team of one."""

    def __init__(self, fabric):
        self.fabric, self.handed_over = fabric, []

    def _native_team(self):
        f = self.fabric
        return (f.engine(), f.comm_stream.cuda_stream, f.device.index, f.overlap_blocks, [0])

    def _native_failed(self):
        self.fabric.check()

    def shutdown(self):
        pass

    def __getattr__(self, name):            # any collective that is handed over is recorded
        def handed(*args):
            self.handed_over.append(name)
            return None
        return handed


def test_one_rank_native_path():
    import torch.distributed as dist
    from gpubridge_b200.ops import _build_c10d, fabric as fabric_mod
    dev = torch.device("cuda", 0)
    fabric = fabric_mod.create_single(dev)
    group = _OneRankGroup(fabric)
    backend = _build_c10d.load().GbBackend(0, 1, group)
    try:
        for dtype in (torch.float32, torch.bfloat16, torch.int64):
            for n in (1, 4099, (1 << 20) + 5, (9 << 20) + 3):
                # the producer runs on a side stream: the collective must wait for it
                side = torch.cuda.Stream(dev)
                with torch.cuda.stream(side):
                    t = torch.zeros(n, dtype=dtype, device=dev)
                    torch.cuda._sleep(2_000_000)
                    t += 3
                    opts = dist.AllreduceOptions()
                    opts.reduceOp = dist.ReduceOp.SUM
                    work = backend.allreduce([t], opts)
                    work.wait()                   # orders the side stream behind the kernel
                    out = t * 2
                side.synchronize()
                assert torch.equal(out.cpu(), torch.full((n,), 6, dtype=dtype)), (dtype, n)
                assert work.is_completed() and work.result()[0] is not None
        t = torch.arange(1000, dtype=torch.float32, device=dev)
        opts = dist.AllreduceOptions()
        opts.reduceOp = dist.ReduceOp.AVG
        fut = backend.allreduce([t], opts).get_future()
        doubled = fut.then(lambda f: f.value()[0] * 2)
        assert torch.equal(doubled.wait().cpu(), torch.arange(1000.) * 2)
        out = torch.empty(777, device=dev)
        backend._allgather_base(out, torch.arange(777., device=dev)).wait()
        assert torch.equal(out.cpu(), torch.arange(777.))
        out = torch.empty(555, device=dev)
        backend._reduce_scatter_base(out, torch.arange(555., device=dev)).wait()
        assert torch.equal(out.cpu(), torch.arange(555.))
        b = torch.arange(100., device=dev)
        backend.broadcast([b]).wait()
        assert torch.equal(b.cpu(), torch.arange(100.))
        torch.cuda.synchronize(dev)
        assert backend.native_calls == 12 + 4 and backend.fallback_calls == 0 and not group.handed_over
        # what the engine does not take is handed over: CPU tensors, unsupported ops
        backend.allreduce([torch.ones(3)])
        opts = dist.AllreduceOptions()
        opts.reduceOp = dist.ReduceOp.PRODUCT
        backend.allreduce([torch.ones(3, device=dev)], opts)
        assert group.handed_over == ["allreduce", "allreduce"] and backend.fallback_calls == 2
        fabric.check()
    finally:
        backend.forget()
        torch.cuda.synchronize(dev)
        fabric.close()


def _through_the_backend(rank, world):
    import torch.distributed as dist
    import gpubridge_b200.native_backend as nb
    dev = torch.device("cuda", rank)
    for dtype in (torch.float32, torch.bfloat16, torch.int32):
        for n in (1, 4099, (1 << 20) + 5, (6 << 20) + 1):
            t = rank_tensor(rank, n, dtype).to(dev)
            dist.all_reduce(t)
            assert torch.equal(t.cpu(), expected_sum(world, n, dtype)), (dtype, n)
    n = 100_003
    t = rank_tensor(rank, n).to(dev)
    dist.all_reduce(t, op=dist.ReduceOp.AVG)
    assert torch.equal(t.cpu(), expected_sum(world, n) / world)
    out = torch.empty(world * n, device=dev)
    dist.all_gather_into_tensor(out, rank_tensor(rank, n).to(dev))
    assert torch.equal(out.cpu(), torch.cat([rank_tensor(r, n) for r in range(world)]))
    out = torch.empty(n, device=dev)
    dist.reduce_scatter_tensor(out, rank_tensor(rank, world * n).to(dev))
    assert torch.equal(out.cpu(), expected_sum(world, world * n).view(world, n)[rank])
    b = rank_tensor(rank, n).to(dev)
    dist.broadcast(b, world - 1)
    assert torch.equal(b.cpu(), rank_tensor(world - 1, n))
    backend = nb.backend_of()
    assert backend.native_calls >= 16, (backend.native_calls, backend.fallback_calls)
    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(32, 64), torch.nn.ReLU(), torch.nn.Linear(64, 8)).to(dev)
    ddp = torch.nn.parallel.DistributedDataParallel(model, device_ids=[rank])
    opt = torch.optim.SGD(ddp.parameters(), lr=0.1)
    torch.manual_seed(100 + rank)
    for _ in range(3):
        opt.zero_grad()
        ddp(torch.randn(16, 32, device=dev)).square().mean().backward()
        opt.step()
    flat = torch.cat([p.detach().reshape(-1) for p in model.parameters()])
    hi, lo = flat.clone(), flat.clone()
    dist.all_reduce(hi, op=dist.ReduceOp.MAX)
    dist.all_reduce(lo, op=dist.ReduceOp.MIN)
    assert torch.equal(hi, lo), "replicas diverged"
    return True


# Not yet run on several GPUs: joins the suite on request until it has.
@pytest.mark.skipif(NGPU < 2 or os.environ.get("GPUBRIDGE_TEST_NATIVE_BACKEND") != "1",
                    reason="needs two GPUs and GPUBRIDGE_TEST_NATIVE_BACKEND=1")
@pytest.mark.parametrize("split", [{}, {"GPUBRIDGE_SPLIT_TEST": "half"}])
def test_backend_end_to_end(tmp_path, split):
    world = 8 if NGPU >= 8 else 4 if NGPU >= 4 else 2
    run_ranks(gpu_ranks(world), _through_the_backend, tmp_path, mode="native-backend",
              env={**split, "GPUBRIDGE_WAIT_TIMEOUT_MS": "10000"}, timeout=240)
