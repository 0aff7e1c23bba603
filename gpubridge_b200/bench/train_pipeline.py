"""Pipeline-parallel training over ``backend="gpubridge"``: a Llama model cut into contiguous
stages, one per rank, driven by ``torch.distributed.pipelining`` (GPipe or 1F1B).  Activations
go forward and their gradients back through the backend's point-to-point sends: NCCL between
GPUs of one box, the host-staged engine between islands in simulation or across hosts.

    python -m torch.distributed.run --nproc-per-node 4 --master-addr 127.0.0.1 \
        -m gpubridge_b200.bench.train_pipeline --model llama-125m --schedule 1f1b --split auto
    GPUBRIDGE_VENDOR=nvidia GPUBRIDGE_SPLIT_TEST=half python -m torch.distributed.run \
        --nproc-per-node 2 --master-addr 127.0.0.1 -m gpubridge_b200.bench.train_pipeline \
        --model llama-tiny --steps 6 --json /tmp/pp.json                  # CPU simulation

``--split``: ``even`` (default), explicit blocks per stage (``7,5``), or ``auto``: every rank
profiles each block on its own device, neighbouring stages time their link, and
:mod:`gpubridge_b200.balance` picks the contiguous split whose slowest stage - transfers
included - is fastest within each device's memory.  ``--backend gloo`` runs the same pipeline
on a plain Gloo group; the losses must match bit for bit on CPU.

Rank 0 writes ``--json``: the loss of every step (mean over microbatches, from the last
stage), the step times (slowest stage), tokens/s from the median step after warm-up, each
stage's blocks and, for ``auto``, the profile and the predicted stage times.  Counterpart of
the reference's ``scripts/gpu/train_pipeline.py`` and ``docs/PIPELINE.md``.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import time
import warnings
from datetime import timedelta
from pathlib import Path

import torch
import torch.distributed as dist
import torch.nn.functional as F
from torch import nn

import gpubridge_b200 as gb
from gpubridge_b200 import balance
from gpubridge_b200.models import llama

SCHEDULES = ("gpipe", "1f1b")


def even_split(blocks: int, stages: int) -> list[int]:
    if blocks < stages:
        raise ValueError(f"{blocks} blocks cannot give each of {stages} stages one")
    base, extra = divmod(blocks, stages)
    return [base + (s < extra) for s in range(stages)]


class BlockWithRope(nn.Module):
    """A transformer block that builds its own rotary tables, so stages (and the profiler)
    can call blocks with one tensor."""

    def __init__(self, block: nn.Module, config) -> None:
        super().__init__()
        self.block, self.config = block, config

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        c = self.config
        cos, sin = llama.rope_tables(c.width // c.heads, x.shape[1], c.rope_base, x.device)
        return self.block(x, cos, sin)


class Stage(nn.Module):
    """Blocks ``[lo, hi)`` plus the embedding on the first stage and the final norm and the
    output layer on the last."""

    def __init__(self, model: llama.Llama, lo: int, hi: int, first: bool, last: bool) -> None:
        super().__init__()
        self.embed = model.embed if first else None
        self.blocks = nn.ModuleList(BlockWithRope(b, model.config) for b in model.blocks[lo:hi])
        self.norm = model.norm if last else None
        self.head = model.head if last else None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.embed is not None:
            x = self.embed(x)
        for block in self.blocks:
            x = block(x)
        if self.head is not None:
            x = self.head(self.norm(x))
        return x


def token_loss(logits: torch.Tensor, target: torch.Tensor) -> torch.Tensor:
    return F.cross_entropy(logits.reshape(-1, logits.shape[-1]).float(), target.reshape(-1))


def everyone(value):
    out = [None] * dist.get_world_size()
    dist.all_gather_object(out, value)
    return out


def link_bytes_per_ms(rank: int, world: int, device: torch.device, nbytes: int) -> list[float]:
    """Bandwidth of each link stage s -> s+1, timed with a send of ``nbytes`` each way."""
    payload = torch.zeros(max(1, nbytes // 4), device=device)
    rates = []
    for s in range(world - 1):
        seconds = 0.0
        if rank in (s, s + 1):
            peer = s + 1 if rank == s else s
            for trial in range(3):
                if device.type == "cuda":
                    torch.cuda.synchronize(device)
                t0 = time.perf_counter()
                if rank == s:
                    dist.send(payload, peer)
                    dist.recv(payload, peer)
                else:
                    dist.recv(payload, peer)
                    dist.send(payload, peer)
                if device.type == "cuda":
                    torch.cuda.synchronize(device)
                if trial:
                    seconds = max(seconds, time.perf_counter() - t0) if trial == 1 else min(
                        seconds, time.perf_counter() - t0)
        took = max(everyone(seconds))
        rates.append(2 * payload.numel() * 4 / max(took * 1e3, 1e-6))
        dist.barrier()
    return rates


def auto_split(model: llama.Llama, rank: int, world: int, device: torch.device, micro: int,
               seq: int, schedule: str, microbatches: int) -> tuple[list[int], dict]:
    """Profile on every rank, exchange, and run the exact partitioner (same answer everywhere)."""
    config = model.config
    layers = [BlockWithRope(b, config) for b in model.blocks]
    example = torch.randn(micro, seq, config.width)
    costs = balance.profile_layers(layers, example, device)
    table = everyone([(c.forward_ms + c.backward_ms, c.out_bytes, c.state_bytes,
                       c.activation_bytes) for c in costs])
    layer_ms = [[row[0] for row in per_rank] for per_rank in table]
    boundary = [table[0][i][1] for i in range(len(costs) - 1)]
    rates = link_bytes_per_ms(rank, world, device, table[0][0][1]) if world > 1 else []
    memory = None
    if device.type == "cuda":
        free = everyone(torch.cuda.mem_get_info(device)[0] * 0.8)
        memory = free
    plan = balance.partition(
        layer_ms, boundary, rates,
        state_bytes=[r[2] for r in table[0]] if memory else None,
        activation_bytes=[r[3] for r in table[0]] if memory else None,
        in_flight=balance.in_flight(schedule, world, microbatches) if memory else None,
        memory_bytes=memory)
    return plan.split, {"layer_ms": layer_ms, "boundary_bytes": boundary,
                        "link_bytes_per_ms": rates, "predicted_stage_ms": plan.stage_ms,
                        "predicted_bottleneck_ms": plan.bottleneck_ms}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", default="llama-tiny", choices=sorted(llama.CONFIGS))
    ap.add_argument("--schedule", default="gpipe", choices=SCHEDULES)
    ap.add_argument("--microbatches", type=int, default=4)
    ap.add_argument("--batch", type=int, default=8, help="global batch per step")
    ap.add_argument("--seq", type=int, default=64)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup-steps", type=int, default=2)
    ap.add_argument("--lr", type=float, default=3e-4)
    ap.add_argument("--split", default="even")
    ap.add_argument("--backend", default="gpubridge", choices=("gpubridge", "gloo", "nccl"))
    ap.add_argument("--timeout", type=float, default=600)
    ap.add_argument("--json", type=Path)
    args = ap.parse_args(argv)
    if args.batch % args.microbatches:
        ap.error("--batch must be a multiple of --microbatches")

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    on_gpu = torch.cuda.is_available() and not os.environ.get("GPUBRIDGE_VENDOR")
    device = torch.device("cuda", local) if on_gpu else torch.device("cpu")
    if on_gpu:
        torch.cuda.set_device(device)
    with warnings.catch_warnings():
        warnings.simplefilter("ignore", gb.SplitTestWarning)
        dist.init_process_group(args.backend, timeout=timedelta(seconds=args.timeout))
    dist.barrier()

    from torch.distributed.pipelining import PipelineStage, Schedule1F1B, ScheduleGPipe

    model = llama.build(args.model, seed=0, device="cpu")
    config = model.config
    micro = args.batch // args.microbatches
    profile = None
    if args.split == "auto":
        split, profile = auto_split(model, rank, world, device, micro, args.seq, args.schedule,
                                    args.microbatches)
    elif args.split == "even":
        split = even_split(config.layers, world)
    else:
        split = [int(s) for s in args.split.split(",")]
        if len(split) != world or sum(split) != config.layers or min(split) < 1:
            ap.error(f"--split needs {world} positive counts adding up to {config.layers}")
    lo = sum(split[:rank])
    stage_module = Stage(model, lo, lo + split[rank], rank == 0, rank == world - 1).to(device)
    del model
    stage = PipelineStage(stage_module, rank, world, device)
    schedule_cls = ScheduleGPipe if args.schedule == "gpipe" else Schedule1F1B
    schedule = schedule_cls(stage, n_microbatches=args.microbatches, loss_fn=token_loss)
    optimizer = torch.optim.AdamW(stage_module.parameters(), lr=args.lr)

    losses, times = [], []
    for step in range(args.steps):
        x, y = llama.synthetic_tokens(config, args.batch, args.seq, seed=step)
        if on_gpu:
            torch.cuda.synchronize(device)
        t0 = time.perf_counter()
        optimizer.zero_grad(set_to_none=True)
        micro_losses: list[torch.Tensor] = []
        if rank == 0:
            schedule.step(x.to(device))
        elif rank == world - 1:
            schedule.step(target=y.to(device), losses=micro_losses)
        else:
            schedule.step()
        optimizer.step()
        if on_gpu:
            torch.cuda.synchronize(device)
        took = time.perf_counter() - t0
        loss = float(torch.stack(micro_losses).mean()) if micro_losses else None
        times.append(max(everyone(took)))
        losses.append(everyone(loss)[world - 1])
    timed = times[args.warmup_steps:] or times
    median = statistics.median(timed)
    record = {"bench": "train_pipeline", "model": args.model, "backend": args.backend,
              "schedule": args.schedule, "stages": world, "split": split,
              "microbatches": args.microbatches, "global_batch": args.batch, "seq": args.seq,
              "losses": losses, "step_ms": [round(t * 1e3, 3) for t in times],
              "median_step_ms": round(median * 1e3, 3),
              "tokens_per_s": round(args.batch * args.seq / median, 1),
              "ideal_bubble_share": round((world - 1) / (args.microbatches + world - 1), 4),
              "profile": profile}
    if rank == 0:
        print(json.dumps({k: v for k, v in record.items() if k not in ("profile", "step_ms")}),
              flush=True)
        if args.json:
            args.json.parent.mkdir(parents=True, exist_ok=True)
            args.json.write_text(json.dumps(record, indent=1))
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
