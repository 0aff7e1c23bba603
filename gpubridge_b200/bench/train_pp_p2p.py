"""Pipeline parallelism the way Megatron-Core drives it: a hand-scheduled 1F1B whose stages talk
only through ``batch_isend_irecv``.

    torchrun --nproc-per-node 4 -m gpubridge_b200.bench.train_pp_p2p --model llama-350m \\
        --microbatches 8 --batch 16 --seq 1024 --json pp_p2p.json
    GPUBRIDGE_VENDOR=nvidia GPUBRIDGE_SPLIT_TEST=half torchrun --nproc-per-node 2 \\
        -m gpubridge_b200.bench.train_pp_p2p --model llama-tiny --verify          # CPU ranks

What a framework with its own pipeline schedule needs of a backend is small and exact: batched
point-to-point operations that may pair a send with a receive to the same neighbour in one
batch (so neither side's send waits behind its own receive), tensors of a shape both sides
know, and completion handles.  This program uses the backend exactly so - the four combined
operations of Megatron-Core's ``p2p_communication`` (receive forward; send forward and receive
backward; send backward and receive forward; send backward) - with every rank one stage
(Llama blocks split evenly, embedding on the first stage, final norm and output layer on the
last), the warm-up / steady 1F1B / cool-down schedule, and AdamW per stage.  It stands in for
the reference's ``scripts/gpu/megatron_pp.py`` (Megatron-Core itself is not a dependency).

``--verify`` replays the same global batch in one process on rank 0 and checks the loss of every
step against it.  Rank 0 writes ``--json``: losses, step times, tokens/s from the median step.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import time
import warnings
from pathlib import Path

import torch
import torch.distributed as dist

import gpubridge_b200 as gb
from gpubridge_b200.bench.train_pipeline import Stage, even_split, token_loss
from gpubridge_b200.models import llama


class Neighbours:
    """The four combined operations between a stage and its neighbours."""

    def __init__(self, rank: int, world: int, shape, dtype, device) -> None:
        self.prev = rank - 1 if rank > 0 else None
        self.next = rank + 1 if rank < world - 1 else None
        self.stages_after = world - 1 - rank
        self.shape, self.dtype, self.device = shape, dtype, device
        self.batches = 0

    def _run(self, send_prev=None, send_next=None, recv_prev=False, recv_next=False):
        ops, got_prev, got_next = [], None, None
        if send_prev is not None:
            ops.append(dist.P2POp(dist.isend, send_prev, self.prev))
        if recv_prev:
            got_prev = torch.empty(self.shape, dtype=self.dtype, device=self.device)
            ops.append(dist.P2POp(dist.irecv, got_prev, self.prev))
        if send_next is not None:
            ops.append(dist.P2POp(dist.isend, send_next, self.next))
        if recv_next:
            got_next = torch.empty(self.shape, dtype=self.dtype, device=self.device)
            ops.append(dist.P2POp(dist.irecv, got_next, self.next))
        if ops:
            self.batches += 1
            for work in gb.batch_isend_irecv(ops):
                work.wait()
        return got_prev, got_next

    def recv_forward(self):
        return self._run(recv_prev=True)[0] if self.prev is not None else None

    def send_forward(self, out):
        if self.next is not None:
            self._run(send_next=out)

    def send_forward_recv_backward(self, out):
        return self._run(send_next=out, recv_next=True)[1] if self.next is not None else None

    def send_backward_recv_forward(self, grad):
        return self._run(send_prev=grad, recv_prev=True)[0] if self.prev is not None else None

    def recv_backward(self):
        return self._run(recv_next=True)[1] if self.next is not None else None

    def send_backward(self, grad):
        if self.prev is not None:
            self._run(send_prev=grad)


def one_f_one_b(stage, links: Neighbours, micro_x, micro_y, first: bool, last: bool):
    """One optimizer step's forwards and backwards; returns the mean loss (last stage)."""
    m = len(micro_x)
    warmup = min(m, links.stages_after)         # forwards in flight before the first backward
    inputs, outputs, losses = [], [], []

    def forward(i, received):
        x = micro_x[i] if first else received.requires_grad_()
        out = stage(x)
        if last:
            out = token_loss(out, micro_y[i]) / m
            losses.append(out.detach())
        inputs.append(None if first else x)
        outputs.append(out)
        return out

    def backward(grad):
        x, out = inputs.pop(0), outputs.pop(0)
        if last:
            out.backward()
        else:
            out.backward(grad)
        return None if x is None else x.grad

    received = links.recv_forward()
    for i in range(warmup):
        out = forward(i, received)
        links.send_forward(out.detach())
        if i + 1 < m:
            received = links.recv_forward()
    for i in range(warmup, m):                    # steady state: one forward, one backward
        out = forward(i, received)
        grad = links.send_forward_recv_backward(out.detach()) if not last else None
        grad_in = backward(grad)
        if i + 1 < m:
            received = (links.send_backward_recv_forward(grad_in) if not first else None)
        elif not first:
            links.send_backward(grad_in)
    for _ in range(warmup):                       # cool-down: the backwards still owed
        grad_in = backward(links.recv_backward())
        if not first:
            links.send_backward(grad_in)
    return torch.stack(losses).sum() if last else None


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", default="llama-tiny", choices=sorted(llama.CONFIGS))
    ap.add_argument("--microbatches", type=int, default=4)
    ap.add_argument("--batch", type=int, default=8, help="global batch per step")
    ap.add_argument("--seq", type=int, default=64)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup-steps", type=int, default=2)
    ap.add_argument("--lr", type=float, default=3e-3)
    ap.add_argument("--backend", default="gpubridge", choices=("gpubridge", "gpubridge_native", "gloo", "nccl"))
    ap.add_argument("--verify", action="store_true")
    ap.add_argument("--json", type=Path)
    args = ap.parse_args(argv)
    if args.batch % args.microbatches:
        ap.error("--batch must be a multiple of --microbatches")
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    on_gpu = torch.cuda.is_available() and not os.environ.get("GPUBRIDGE_VENDOR")
    device = torch.device("cuda", local) if on_gpu else torch.device("cpu")
    if on_gpu:
        torch.cuda.set_device(device)
    else:
        torch.set_num_threads(1)
    if args.backend == "gpubridge_native":
        import gpubridge_b200.native_backend  # noqa: F401 - registers the name
    with warnings.catch_warnings():
        warnings.simplefilter("ignore", gb.SplitTestWarning)
        dist.init_process_group(args.backend)
    whole = llama.build(args.model, seed=0, device=device, dtype=torch.float32)
    config = whole.config
    split = even_split(config.layers, world)
    lo = sum(split[:rank])
    first, last = rank == 0, rank == world - 1
    stage = Stage(whole, lo, lo + split[rank], first, last)
    optimizer = torch.optim.AdamW(stage.parameters(), lr=args.lr)
    micro = args.batch // args.microbatches
    links = Neighbours(rank, world, (micro, args.seq, config.width), torch.float32, device)
    oracle = oracle_opt = None
    if args.verify and rank == 0:
        oracle = llama.build(args.model, seed=0, device=device, dtype=torch.float32)
        oracle_opt = torch.optim.AdamW(oracle.parameters(), lr=args.lr)

    def wait():
        if on_gpu:
            torch.cuda.synchronize(device)

    losses, times, worst = [], [], 0.0
    for step in range(args.warmup_steps + args.steps):
        x, y = llama.rule_batch(config, step, args.batch, args.seq)
        x, y = x.to(device), y.to(device)
        wait()
        dist.barrier()
        t0 = time.perf_counter()
        optimizer.zero_grad(set_to_none=True)
        loss = one_f_one_b(stage, links, x.split(micro), y.split(micro), first, last)
        optimizer.step()
        wait()
        took = [None] * world
        dist.all_gather_object(took, (time.perf_counter() - t0, float(loss) if last else None))
        times.append(max(t for t, _ in took))
        losses.append(took[-1][1])
        if oracle is not None:
            oracle_opt.zero_grad(set_to_none=True)
            want = token_loss(oracle(x), y)
            want.backward()
            oracle_opt.step()
            worst = max(worst, abs(float(want.detach()) - losses[-1]))
    median = statistics.median(times[args.warmup_steps:] or times)
    record = {"bench": "train_pipeline", "schedule": "1f1b (batched p2p)", "model": args.model,
              "backend": args.backend, "stages": world, "split": split, "microbatches": args.microbatches,
              "global_batch": args.batch, "seq": args.seq, "losses": losses,
              "step_ms": [round(t * 1e3, 3) for t in times], "median_step_ms": round(median * 1e3, 3),
              "tokens_per_s": round(args.batch * args.seq / median, 1),
              "p2p_batches_per_step": links.batches / len(times),
              "largest_loss_gap_to_one_process": worst if args.verify else None}
    code = 0
    if rank == 0:
        print(json.dumps({k: v for k, v in record.items() if k not in ("losses", "step_ms")}), flush=True)
        if args.json:
            args.json.parent.mkdir(parents=True, exist_ok=True)
            args.json.write_text(json.dumps(record, indent=1))
        if args.verify and not worst < 1e-4:
            print(f"the pipelined loss strayed from the one-process loss by {worst}", file=sys.stderr)
            code = 1
    verdict = [code]
    dist.broadcast_object_list(verdict, src=0)
    dist.destroy_process_group()
    return verdict[0]


if __name__ == "__main__":
    sys.exit(main())
