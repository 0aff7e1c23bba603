"""Where the time of a data-parallel step goes when GPUs are added.

The flagship step (GPT-2 small, 8 x 1024 tokens per GPU, bf16 autocast, AdamW, CUDA graph) is
run through ``DataParallelTrainer`` in several variants on the same ranks, one after another,
each device-timed (CUDA events, barrier and synchronize on both sides, slowest rank):

* ``compute``       - this rank alone (no exchange): the step a lone GPU runs;
* ``default``       - 25 MB buckets, bucket all-reduces beside backward on few CTAs;
* ``exposed``       - one bucket: the whole gradient is averaged after backward on the full
                      grid, nothing overlaps (``exposed - compute`` = the exchange itself);
* ``blocks=N``      - the CTAs a bucket's all-reduce may take beside backward;
* ``bucket=N``      - bucket size in MB.

``default - compute`` is what the exchange costs the step; its lower bound is the part of
``exposed - compute`` that the last bucket accounts for.  ``--timeline`` adds one eager step
with CUDA events around every bucket's all-reduce on the communication stream: when each
starts and ends, relative to the start of the step, and what is left of the step after the last.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        -m gpubridge_b200.bench.ddp_attribution --steps 20 --timeline

Rank 0 prints one JSON object.  (Reference: the comparison its scripts/gpu/train_bench.py makes
between a lone GPU and DDP, without the breakdown.)
"""
from __future__ import annotations

import argparse
import json
import os
import warnings

import torch

BATCH, SEQ = 8, 1024


def _batches(vocab: int, device, seed: int):
    g = torch.Generator().manual_seed(seed)
    out = []
    for _ in range(4):
        tokens = torch.randint(vocab, (BATCH, SEQ + 1), generator=g)
        out.append((tokens[:, :-1].contiguous().to(device), tokens[:, 1:].contiguous().to(device)))
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--blocks", default="8,16,64", help="overlap grids to try")
    ap.add_argument("--buckets", default="10,50,100", help="bucket sizes (MB) to try")
    ap.add_argument("--timeline", action="store_true")
    ap.add_argument("--model", default="gpt2-small")
    args = ap.parse_args(argv)

    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1:
        os.environ.setdefault("GPUBRIDGE_SPLIT_TEST", "half")
    import gpubridge_b200 as gb
    from gpubridge_b200.models import gpt2
    from gpubridge_b200.parallel.trainer import DataParallelTrainer

    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    topology = None
    if world > 1:
        with warnings.catch_warnings():
            warnings.simplefilter("ignore", gb.SplitTestWarning)
            topology = gb.init()
    data = _batches(gpt2.CONFIGS[args.model].vocab, device, seed=rank)

    def barrier() -> None:
        if topology is not None:
            topology.world_group.barrier()

    def slowest(value: float) -> float:
        if topology is None:
            return value
        t = torch.tensor([value], dtype=torch.float64)
        topology.world_group.all_reduce(t, "max")
        return float(t)

    def make(**options):
        torch.manual_seed(0)
        model = gpt2.build(args.model).to(device)
        return DataParallelTrainer(model, lambda m, x, y: m.loss(x, y), topology=topology,
                                   lr=3e-4, autocast=torch.bfloat16, **options)

    def measure(**options) -> float:
        trainer = make(graph=True, **options)
        for i in range(args.warmup):
            trainer.step(*data[i % len(data)])
        torch.cuda.synchronize(device)
        barrier()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for i in range(args.steps):
            trainer.step(*data[i % len(data)])
        end.record()
        torch.cuda.synchronize(device)
        barrier()
        trainer.check()
        ms = slowest(start.elapsed_time(end)) / args.steps
        del trainer
        torch.cuda.empty_cache()
        return round(ms, 3)

    rows = {"compute": measure(exchange=False)}
    if world > 1:
        rows["default"] = measure()
        rows["exposed"] = measure(bucket_mb=1e9)
        for blocks in [int(b) for b in args.blocks.split(",") if b]:
            rows[f"blocks={blocks}"] = measure(overlap_blocks=blocks)
        for mb in [float(b) for b in args.buckets.split(",") if b]:
            rows[f"bucket={mb:g}"] = measure(bucket_mb=mb)
    result = {"what": "ms per step of the data-parallel GPT-2 step, by variant", "world": world,
              "islands": [len(i.ranks) for i in topology.layout.islands] if topology is not None else None,
              "model": args.model, "steps": args.steps, "ms_per_step": rows}
    if world > 1:
        result["exchange_cost_ms"] = round(rows["default"] - rows["compute"], 3)
        result["exchange_alone_ms"] = round(rows["exposed"] - rows["compute"], 3)
        fabric = topology.fabric
        result["in_switch_reduction"] = bool(fabric is not None and fabric.sw_team is not None)

    if args.timeline and world > 1 and topology.fabric is not None:
        result["timeline"] = _timeline(make(graph=False), data, topology, device, barrier)
    if topology is not None:
        gb.destroy()
    if rank == 0:
        print(json.dumps(result))
    return 0


def _timeline(trainer, data, topology, device, barrier) -> dict:
    """One eager step with events around each bucket's all-reduce (this rank's clock)."""
    comm = topology.fabric.comm_stream
    marks: list[tuple] = []
    plain = trainer._all_reduce

    def traced(grads, tail=False):
        first, last = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        comm.wait_stream(torch.cuda.current_stream(device))
        first.record(comm)
        plain(grads, tail)
        last.record(comm)
        marks.append((first, last, grads.nbytes, tail))

    for i in range(3):
        trainer.step(*data[i % len(data)])
    trainer._all_reduce = traced
    torch.cuda.synchronize(device)
    barrier()
    marks.clear()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    trainer.step(*data[0])
    end.record()
    torch.cuda.synchronize(device)
    barrier()
    buckets = [{"mb": round(nbytes / 2**20, 1), "tail": bool(tail),
                "start_ms": round(start.elapsed_time(first), 3),
                "end_ms": round(start.elapsed_time(last), 3)}
               for first, last, nbytes, tail in marks]
    busy = sum(b["end_ms"] - b["start_ms"] for b in buckets)
    return {"eager_step_ms": round(start.elapsed_time(end), 3), "buckets": buckets,
            "comm_stream_busy_ms": round(busy, 3),
            "after_last_bucket_ms": round(start.elapsed_time(end) - buckets[-1]["end_ms"], 3)
            if buckets else None}


if __name__ == "__main__":
    raise SystemExit(main())
