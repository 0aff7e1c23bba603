"""Data-parallel training throughput of the Llama-style models through backend="gpubridge":
``ddp``, ``fsdp2`` (``fully_shard`` on a 1-D mesh) and ``hsdp`` (shard inside an island,
replicate across islands; the cross-island gradient all-reduce is the compressed one when
``GPUBRIDGE_BRIDGE_COMPRESSION`` is set).  Counterpart of the reference's
scripts/gpu/train_dp.py.

    GPUBRIDGE_ISLANDS=4,4 GPUBRIDGE_BRIDGE_COMPRESSION=fp8 GPUBRIDGE_CODEC_FORMAT=b200 \
      python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 \
      -m gpubridge_b200.bench.train_dp --model llama3-8b --mode hsdp --batch 1 --seq 4096

Timing: warm-up steps, then ``--steps`` steps between CUDA events with a barrier and a
synchronize on both sides; the slowest rank counts.  One JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
import warnings

import torch
import torch.distributed as dist

import gpubridge_b200 as gb
from gpubridge_b200.models import llama


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--model", default="llama-125m", choices=sorted(llama.CONFIGS))
    ap.add_argument("--mode", default="fsdp2", choices=("single", "ddp", "fsdp2", "hsdp"))
    ap.add_argument("--batch", type=int, default=4)
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--lr", type=float, default=3e-4)
    ap.add_argument("--backend", default="gpubridge", help="gpubridge or nccl (the baseline)")
    ap.add_argument("--rng", default="device", choices=("cpu", "device"),
                    help="where the random initial weights are drawn (same seed on every rank)")
    args = ap.parse_args(argv)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    on_gpu = torch.cuda.is_available() and not os.environ.get("GPUBRIDGE_VENDOR")
    device = torch.device("cuda", local) if on_gpu else torch.device("cpu")
    if on_gpu:
        torch.cuda.set_device(device)
    with warnings.catch_warnings():
        warnings.simplefilter("ignore", gb.SplitTestWarning)
        dist.init_process_group(args.backend if on_gpu or args.backend == "gpubridge" else "gloo")
    dtype = torch.bfloat16 if on_gpu else torch.float32
    model = llama.build(args.model, seed=0, device=device, dtype=torch.float32, rng=args.rng)
    config = model.config
    if args.mode == "ddp":
        from torch.nn.parallel import DistributedDataParallel as DDP
        model = DDP(model, device_ids=[local] if on_gpu else None)
    elif args.mode in ("fsdp2", "hsdp"):
        from torch.distributed.device_mesh import init_device_mesh
        from torch.distributed.fsdp import MixedPrecisionPolicy, fully_shard
        kind = "cuda" if on_gpu else "cpu"
        if args.mode == "hsdp":
            islands = [int(s) for s in os.environ.get("GPUBRIDGE_ISLANDS", "").split(",") if s]
            shard = islands[0] if islands else max(1, world // 2)
            mesh = init_device_mesh(kind, (world // shard, shard),
                                    mesh_dim_names=("replicate", "shard"))
        else:
            mesh = init_device_mesh(kind, (world,))
        policy = MixedPrecisionPolicy(param_dtype=dtype, reduce_dtype=dtype) if on_gpu else \
            MixedPrecisionPolicy()
        for block in model.blocks:
            fully_shard(block, mesh=mesh, mp_policy=policy)
        fully_shard(model, mesh=mesh, mp_policy=policy)
    optimizer = torch.optim.AdamW(model.parameters(), lr=args.lr, fused=on_gpu)
    x, y = llama.synthetic_tokens(config, args.batch, args.seq, seed=0 + rank)
    x, y = x.to(device), y.to(device)
    core = model.module if hasattr(model, "module") else model

    def step() -> torch.Tensor:
        optimizer.zero_grad(set_to_none=True)
        if args.mode in ("single", "ddp") and on_gpu:
            with torch.autocast("cuda", dtype=dtype):
                logits = model(x)
        else:
            logits = model(x)
        loss = torch.nn.functional.cross_entropy(logits.view(-1, logits.shape[-1]).float(),
                                                 y.reshape(-1))
        loss.backward()
        optimizer.step()
        return loss.detach()

    for _ in range(args.warmup):
        loss = step()
    if on_gpu:
        torch.cuda.synchronize(device)
    dist.barrier()
    sampler = None
    if on_gpu:
        from gpubridge_b200.utils import ClockSampler
        sampler = ClockSampler(local)
        sampler.start()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        loss = step()
    if on_gpu:
        end.record()
        torch.cuda.synchronize(device)
        ms = start.elapsed_time(end)
    else:
        ms = (time.perf_counter() - t0) * 1e3
    clocks = sampler.stop() if sampler is not None else None
    dist.barrier()
    slowest = torch.tensor([ms], dtype=torch.float64, device=device)
    dist.all_reduce(slowest, op=dist.ReduceOp.MAX)
    tokens = args.batch * args.seq * world * args.steps
    if rank == 0:
        topology = gb.get_topology() if gb.is_initialized() else None
        print(json.dumps({
            "bench": "train_dp", "model": args.model, "mode": args.mode, "backend": args.backend,
            "world": world, "islands": [len(i.ranks) for i in topology.layout.islands] if topology else None,
            "batch_per_gpu": args.batch, "seq": args.seq, "steps": args.steps,
            "ms_per_step": round(float(slowest) / args.steps, 3),
            "tokens_per_s": round(tokens / (float(slowest) * 1e-3), 1),
            "loss": round(float(loss), 4),
            "compression": os.environ.get("GPUBRIDGE_BRIDGE_COMPRESSION", ""),
            "parameters": sum(p.numel() for p in core.parameters()),
            "clocks": clocks,
        }), flush=True)
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
