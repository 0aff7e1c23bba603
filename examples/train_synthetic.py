"""Data-parallel training on synthetic data; throughput and a bit-for-bit sync check.

    torchrun --nproc-per-node 8 examples/train_synthetic.py --json results/scaling/train-n8.json
    GPUBRIDGE_VENDOR=nvidia torchrun --nproc-per-node 2 examples/train_synthetic.py   # CPU

A small MLP learns a fixed random classification task; every rank trains on its own batches.
``--engine ddp`` (default) wraps the model in DistributedDataParallel with
``gpubridge_b200.ddp_comm_hook``; ``--engine trainer`` uses the flat-buffer
``DataParallelTrainer`` (fused bucket all-reduce, fused AdamW, CUDA graph on GPUs).  Reports
samples/s over all ranks and checks, outside the timed part, that every rank holds the same
parameters bit for bit; the record names the first step at which gradients or parameters
differed.  ``python -m gpubridge_b200.kit.summarize DIR`` turns a directory of
``train-n<N>.json`` records into a weak-scaling table.
"""
from __future__ import annotations

import argparse
import statistics
import sys
import time
from pathlib import Path

import torch
from torch import nn

import os as _os, sys as _sys
_sys.path.insert(0, _os.path.dirname(_os.path.dirname(_os.path.abspath(__file__))))  # run from a checkout
import gpubridge_b200 as gb  # noqa: E402
from gpubridge_b200.kit import environment, run_info, sync, write_json  # noqa: E402


def make_model(dim: int, layers: int, classes: int) -> nn.Module:
    blocks: list[nn.Module] = []
    for _ in range(layers):
        blocks += [nn.Linear(dim, dim), nn.ReLU()]
    return nn.Sequential(*blocks, nn.Linear(dim, classes))


def same_everywhere(tensors) -> bool:
    flat = torch.cat([t.detach().reshape(-1).double() for t in tensors])
    hi, lo = flat.clone(), flat.clone()
    gb.all_reduce(hi, gb.ReduceOp.MAX)
    gb.all_reduce(lo, gb.ReduceOp.MIN)
    return bool(torch.equal(hi, lo))


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--batch", type=int, default=256, help="samples per rank and step")
    ap.add_argument("--dim", type=int, default=512)
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--classes", type=int, default=16)
    ap.add_argument("--engine", choices=("ddp", "trainer"), default="ddp")
    ap.add_argument("--json", type=Path)
    args = ap.parse_args(argv)

    topology = gb.init()
    rank, world, device = topology.rank, topology.world_size, topology.device
    if device.type == "cpu":
        torch.set_num_threads(1)        # as torchrun does for several ranks: comparable steps
    torch.manual_seed(0)
    model = make_model(args.dim, args.layers, args.classes).to(device)
    teacher = torch.randn(args.dim, args.classes, generator=torch.Generator().manual_seed(1)).to(device)
    data = torch.Generator().manual_seed(100 + rank)

    def batch():
        x = torch.randn(args.batch, args.dim, generator=data).to(device)
        return x, (x @ teacher).argmax(1)

    loss_fn = nn.functional.cross_entropy
    first_grad_diff = first_param_diff = None
    if args.engine == "trainer":
        from gpubridge_b200.parallel.trainer import DataParallelTrainer
        trainer = DataParallelTrainer(model, lambda m, x, y: loss_fn(m(x), y), topology=topology,
                                      lr=1e-3, autocast=None, graph=device.type == "cuda")
        step = lambda x, y: trainer.step(x, y)          # noqa: E731
    else:
        import torch.distributed as dist
        from torch.nn.parallel import DistributedDataParallel
        ddp = DistributedDataParallel(model, device_ids=[device.index] if device.type == "cuda" else None)
        ddp.register_comm_hook(None, gb.ddp_comm_hook)
        opt = torch.optim.AdamW(ddp.parameters(), lr=1e-3)
        assert dist.is_initialized()

        def step(x, y):
            opt.zero_grad(set_to_none=True)
            loss = loss_fn(ddp(x), y)
            loss.backward()
            opt.step()
            return loss.detach()

    times, losses = [], []
    for i in range(args.warmup + args.steps):
        x, y = batch()
        sync(device)
        t0 = time.perf_counter()
        loss = step(x, y)
        sync(device)
        if i >= args.warmup:
            times.append(time.perf_counter() - t0)
        losses.append(float(loss))
        if args.engine == "ddp" and first_grad_diff is None and not same_everywhere(
                [p.grad for p in model.parameters() if p.grad is not None]):
            first_grad_diff = i
        if first_param_diff is None and not same_everywhere(list(model.parameters())):
            first_param_diff = i
    in_sync = same_everywhere(list(model.parameters()))
    median = statistics.median(times)
    record = {"world_size": world, "engine": args.engine, "batch_per_rank": args.batch,
              "samples_per_sec": round(args.batch * world / median, 1),
              "step_ms_median": round(median * 1e3, 3), "loss_first": losses[0],
              "loss_last": losses[-1], "params_in_sync": in_sync,
              "first_gradient_difference": first_grad_diff,
              "first_parameter_difference": first_param_diff,
              "run": run_info(topology), "environment": environment()}
    if rank == 0:
        print(f"{world} ranks ({args.engine}): {record['samples_per_sec']} samples/s, median step "
              f"{record['step_ms_median']} ms, loss {losses[0]:.3f} -> {losses[-1]:.3f}, "
              f"parameters {'in sync' if in_sync else 'DIFFER'}")
        if args.json:
            write_json(args.json, record)
    gb.destroy()
    return 0 if in_sync and losses[-1] < losses[0] else 1


if __name__ == "__main__":
    sys.exit(main())
