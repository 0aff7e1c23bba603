"""DataParallelTrainer computes the update that stock PyTorch computes.

The trainer (flat buffers, fused cross-entropy / LayerNorm / AdamW, bucketed fused all-reduce,
optional CUDA graph) is started from the same weights and fed the same data as the plain recipe
it replaces - ``DistributedDataParallel`` with ``gpubridge_b200.ddp_comm_hook`` (one GPU: no
DDP) and ``torch.optim.AdamW`` on stock ``F.cross_entropy`` - and after ten steps the loss
curves and the parameters must agree: tightly in fp32, within bf16 rounding under autocast.
One GPU runs in this process; two or more as one process per GPU on two islands."""
import copy

import pytest
import torch
import torch.nn.functional as F

from _harness import gpu_ranks, run_ranks

pytestmark = pytest.mark.gpu
NGPU = torch.cuda.device_count() if torch.cuda.is_available() else 0
STEPS = 10


def _batches(rank, vocab, count=STEPS, batch=4, seq=32):
    g = torch.Generator().manual_seed(500 + rank)
    tokens = torch.randint(vocab, (count, batch, seq + 1), generator=g)
    return tokens[:, :, :-1].contiguous(), tokens[:, :, 1:].contiguous()


def _compare(rank, topology, autocast, graph):
    """Both recipes on this rank, one after the other; returns (largest loss gap, relative
    distance of the parameters)."""
    from gpubridge_b200.models import gpt2
    from gpubridge_b200.parallel.trainer import DataParallelTrainer
    import gpubridge_b200 as gb
    dev = torch.device("cuda", rank if topology is not None else 0)
    torch.cuda.set_device(dev)
    torch.manual_seed(11)
    ours = gpt2.build("gpt2-tiny").to(dev)
    stock = copy.deepcopy(ours)
    start = torch.cat([p.detach().float().reshape(-1) for p in stock.parameters()]).clone()
    vocab = ours.config.vocab
    xs, ys = _batches(rank, vocab)
    xs, ys = xs.to(dev), ys.to(dev)

    trainer = DataParallelTrainer(ours, lambda m, x, y: m.loss(x, y), topology=topology, lr=1e-3,
                                  autocast=autocast, graph=graph, graph_warmup=2, bucket_mb=0.05)
    mine = [float(trainer.step(xs[i], ys[i])) for i in range(STEPS)]
    trainer.check()

    net = stock
    if topology is not None:
        from torch.nn.parallel import DistributedDataParallel as DDP
        net = DDP(stock, device_ids=[dev.index], bucket_cap_mb=0.05)
        net.register_comm_hook(None, gb.ddp_comm_hook)
    optimizer = torch.optim.AdamW(net.parameters(), lr=1e-3)
    theirs = []
    for i in range(STEPS):
        optimizer.zero_grad(set_to_none=True)
        if autocast is not None:
            with torch.autocast("cuda", dtype=autocast):
                logits = net(xs[i])
        else:
            logits = net(xs[i])
        loss = F.cross_entropy(logits.reshape(-1, vocab).float(), ys[i].reshape(-1))
        loss.backward()
        optimizer.step()
        theirs.append(float(loss))
    a = torch.cat([p.detach().float().reshape(-1) for p in ours.parameters()])
    b = torch.cat([p.detach().float().reshape(-1) for p in stock.parameters()])
    gap = max(abs(x - y) for x, y in zip(mine, theirs))
    distance = float((a - b).norm() / b.norm())
    assert float((b - start).norm()) > 0, "the stock loop did not train"
    return gap, distance


@pytest.mark.parametrize("autocast,graph,loss_tol,param_tol", [
    (None, False, 2e-4, 2e-3), (None, True, 2e-4, 2e-3), (torch.bfloat16, True, 5e-2, 5e-2)],
    ids=["fp32-eager", "fp32-graph", "bf16-graph"])
def test_one_gpu_trainer_equals_the_stock_loop(autocast, graph, loss_tol, param_tol):
    gap, distance = _compare(0, None, autocast, graph)
    assert gap < loss_tol and distance < param_tol, (gap, distance)


def _ranked(rank, topology, autocast, graph):
    return _compare(rank, topology, autocast, graph)


@pytest.mark.skipif(NGPU < 2, reason="needs at least two GPUs")
@pytest.mark.parametrize("autocast,graph,loss_tol,param_tol", [
    (None, False, 2e-4, 2e-3), (torch.bfloat16, True, 5e-2, 5e-2)], ids=["fp32-eager", "bf16-graph"])
def test_trainer_equals_ddp_with_the_hook(tmp_path, autocast, graph, loss_tol, param_tol):
    world = 4 if NGPU >= 4 else 2
    out = run_ranks(gpu_ranks(world), _ranked, tmp_path, autocast, graph,
                    env={"GPUBRIDGE_SPLIT_TEST": "half"}, timeout=240)
    for gap, distance in out:
        assert gap < loss_tol and distance < param_tol, out
