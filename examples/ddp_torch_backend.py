"""DistributedDataParallel over ``backend="gpubridge"``: a stock DDP script apart from the
backend name and the import that registers it.

    torchrun --nproc-per-node 8 examples/ddp_torch_backend.py
    GPUBRIDGE_VENDOR=nvidia GPUBRIDGE_SPLIT_TEST=half torchrun --nproc-per-node 4 \
        examples/ddp_torch_backend.py                      # CPU simulation, two islands

Exits non-zero if the ranks' parameters differ at the end.
"""
from __future__ import annotations

import argparse
import json
import os
from pathlib import Path

import torch
import torch.distributed as dist
from torch import nn
from torch.nn.parallel import DistributedDataParallel

import os as _os, sys as _sys
_sys.path.insert(0, _os.path.dirname(_os.path.dirname(_os.path.abspath(__file__))))  # run from a checkout
import gpubridge_b200  # noqa: F401  registers the backend


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--json", type=Path)
    args = ap.parse_args()
    dist.init_process_group(backend="gpubridge")
    rank, world = dist.get_rank(), dist.get_world_size()
    on_gpu = torch.cuda.is_available() and not os.environ.get("GPUBRIDGE_VENDOR")
    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0))) if on_gpu else torch.device("cpu")
    if on_gpu:
        torch.cuda.set_device(device)
    torch.manual_seed(0)
    model = nn.Sequential(nn.Linear(32, 64), nn.GELU(), nn.Linear(64, 8)).to(device)
    ddp = DistributedDataParallel(model, device_ids=[device.index] if on_gpu else None)
    opt = torch.optim.SGD(ddp.parameters(), lr=0.05)
    teacher = torch.randn(32, 8, generator=torch.Generator().manual_seed(1)).to(device)
    batches = torch.Generator().manual_seed(100 + rank)       # each rank its own data
    losses = []
    for _ in range(args.steps):
        x = torch.randn(64, 32, generator=batches).to(device)
        loss = nn.functional.cross_entropy(ddp(x), (x @ teacher).argmax(1))
        loss.backward()
        opt.step()
        opt.zero_grad()
        losses.append(loss.item())
    same = True
    for p in model.parameters():
        hi, lo = p.detach().clone(), p.detach().clone()
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        same &= bool(torch.equal(hi, lo))
    if rank == 0:
        print(f"{world} ranks: loss {losses[0]:.3f} -> {losses[-1]:.3f}; parameters "
              f"{'identical' if same else 'DIFFER'} on every rank")
        if args.json:
            args.json.parent.mkdir(parents=True, exist_ok=True)
            args.json.write_text(json.dumps({"world": world, "losses": losses, "identical": same}))
    dist.destroy_process_group()
    return 0 if same else 1


if __name__ == "__main__":
    raise SystemExit(main())
