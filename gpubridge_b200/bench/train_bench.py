"""Data-parallel training throughput on a real model, taken apart into compute, waiting and
gradient exchange.

    torchrun --nproc-per-node 8 -m gpubridge_b200.bench.train_bench --model gpt2-small --json out.json
    GPUBRIDGE_VENDOR=nvidia GPUBRIDGE_SPLIT_TEST=half torchrun --nproc-per-node 2 \\
        -m gpubridge_b200.bench.train_bench --model tiny-gpt            # CPU ranks

The counterpart of the reference's ``scripts/gpu/train_bench.py`` (its method: lines 13-36,
batch splitting 41-68, the native control 70-78, parameter agreement 84-91).

Models (``gpubridge_b200.models``), on synthetic data that each rank draws for itself:
``gpt2-small`` (124 M parameters, next-token loss on random tokens), ``resnet50`` (25.6 M,
random 224x224 images, 1000 classes), and ``tiny-gpt`` / ``tiny-resnet`` for CPU tests.

Engines (``--engine``):

* ``ddp``: ``DistributedDataParallel`` with ``gpubridge_b200.ddp_comm_hook`` - every
  gradient bucket is averaged by an asynchronous ``all_reduce`` beside the rest of backward.
  ``--grad-sync native`` is the control: plain DDP on a group of torch's own backend (NCCL;
  Gloo on CPU, where the record says that it is a stand-in), nothing of this library in the
  gradient path.
* ``trainer``: ``gpubridge_b200.parallel.DataParallelTrainer`` - flat fp32 parameter and
  gradient buffers, stream-ordered fused bucket all-reduces on few CTAs beside backward,
  fused AdamW, and the whole step replayed from a CUDA graph (``--no-graph`` to run it
  eagerly).  The default on GPUs.

Three phases, each step bracketed by a device synchronisation and timed on every rank (CUDA
events on a GPU):

1. **compute** - forward, backward and AdamW with no gradient exchange: this rank alone.
2. **ddp** - the same steps with the exchange.  Ranks start from rank 0's parameters.
3. **comm alone** - the gradient buckets of phase 2, all-reduced the same way with nothing
   beside them.

From the medians (a phase-2 step costs what its slowest rank took):

    compute_ms        this rank's phase 1
    waiting_ms        the slowest rank's compute less this rank's
    exposed_comm_ms   the ddp step less the slowest rank's compute
    hidden_comm_ms    comm alone less the exposed part, at least 0
    samples_per_s     global batch / ddp step;  alone_samples_per_s = batch / compute

The split is a model: compute measured alone differs a little from compute that shares
the GPU with collectives, and the difference lands in ``exposed_comm_ms``.

Batches: ``--batch-size`` per rank (default), ``--batch-sizes a,b,...`` in rank order, or
``--global-batch N`` split evenly - with ``--balance``, split by speed after a calibration
(``--calibration-batch``, ``--calibration-steps``): every further sample goes to the rank
whose predicted compute stays lowest.  With unequal batches each rank weights its loss by
``batch * world / N`` so that the plain average over ranks is the mean over all N samples.
``--accumulate K`` cuts each rank's batch into K micro-batches and exchanges gradients once,
in the last backward.

``--controlled``: fp32 without TF32, deterministic algorithms, digests of the inputs and of
the initial parameters in the record, and the seeded model is rebuilt after phase 1 so that
phase 2 starts from exactly the seeded weights (checked).

After phase 2 the record holds ``params_identical`` (every rank hashes its parameters) and
``params_sum_spread``; a non-finite parameter fails the run.  On a GPU ``memory`` has the
caching allocator's peaks and retries for each phase.  Rank 0 writes ``--json``.
"""
from __future__ import annotations

import argparse
import contextlib
import hashlib
import heapq
import os
import statistics
import sys
import time
from datetime import timedelta
from pathlib import Path

import torch
import torch.distributed as dist
from torch import nn

import gpubridge_b200 as gb
from gpubridge_b200.kit import environment, run_info, sync, write_json
from gpubridge_b200.models import gpt2, resnet

#: name -> (family, config name in the model module, default batch per rank, default sequence)
WORKLOADS = {
    "gpt2-small": ("gpt", "gpt2-small", 8, 1024),
    "tiny-gpt": ("gpt", "gpt2-tiny", 4, 16),
    "resnet50": ("resnet", "resnet50", 64, None),
    "tiny-resnet": ("resnet", "resnet-tiny", 4, None),
}


# -- batches ---------------------------------------------------------------------------------------
def even_shares(total: int, world: int) -> list[int]:
    """``total`` samples over ``world`` ranks; the first ``total % world`` ranks take one more."""
    if total < world:
        raise ValueError(f"{total} samples cannot give each of {world} ranks one")
    base, extra = divmod(total, world)
    return [base + (r < extra) for r in range(world)]


def speed_shares(total: int, seconds_per_sample: list[float], floor: int = 1) -> list[int]:
    """``total`` whole samples, at least ``floor`` per rank, so that the slowest predicted
    compute is as low as whole samples allow: a heap keyed by the time a rank would take
    with one more sample hands out the samples one by one (ties to the lower rank)."""
    world = len(seconds_per_sample)
    if total < floor * world:
        raise ValueError(f"{total} samples cannot give each of {world} ranks {floor}")
    if min(seconds_per_sample) <= 0:
        raise ValueError(f"seconds per sample must be positive: {seconds_per_sample}")
    shares = [floor] * world
    heap = [((floor + 1) * t, r) for r, t in enumerate(seconds_per_sample)]
    heapq.heapify(heap)
    for _ in range(total - floor * world):
        _, r = heapq.heappop(heap)
        shares[r] += 1
        heapq.heappush(heap, ((shares[r] + 1) * seconds_per_sample[r], r))
    return shares


def cut(batch: int, pieces: int) -> list[int]:
    return even_shares(batch, pieces)


class Workload:
    """A model family: how to build it, draw a batch and weight its loss."""

    def __init__(self, name: str, seq: int | None, device: torch.device, controlled: bool) -> None:
        self.family, self.config_name, self.default_batch, default_seq = WORKLOADS[name]
        self.name, self.device, self.controlled = name, device, controlled
        module = gpt2 if self.family == "gpt" else resnet
        self.config = module.CONFIGS[self.config_name]
        self.seq = min(seq or default_seq, self.config.context) if self.family == "gpt" else None
        self.channels_last = self.family == "resnet" and device.type == "cuda" and not controlled
        self.autocast = torch.bfloat16 if device.type == "cuda" and not controlled else None

    def build(self) -> nn.Module:
        torch.manual_seed(0)
        model = (gpt2.build if self.family == "gpt" else resnet.build)(self.config_name).to(self.device)
        return model.to(memory_format=torch.channels_last) if self.channels_last else model

    def data(self, batch: int, rank: int, count: int = 4):
        if self.family == "gpt":
            pairs = gpt2.synthetic_tokens(self.config, batch, self.seq, seed=100 + rank, count=count)
        else:
            pairs = resnet.synthetic_images(self.config, batch, seed=100 + rank, count=count)
        out = []
        for x, y in pairs:
            x = x.to(self.device)
            if self.channels_last:
                x = x.contiguous(memory_format=torch.channels_last)
            out.append((x, y.to(self.device)))
        return out

    def loss_fn(self, per_sample_weight: float | None):
        """``loss_fn(model, x, y)``: the mean over the batch, or with a weight (world / N) the
        sum over the batch's samples times that weight."""
        def loss(model, x, y):
            value = model.loss(x, y)
            return value if per_sample_weight is None else value * (x.shape[0] * per_sample_weight)
        return loss


def digest(tensors) -> str:
    h = hashlib.sha256()
    for t in tensors:
        h.update(t.detach().to("cpu", torch.float32).contiguous().numpy().tobytes())
    return h.hexdigest()[:16]


# -- steppers --------------------------------------------------------------------------------------
class Stepper:
    """``run(micro_batches)`` performs one optimizer step; ``buckets`` lists the byte sizes of
    the gradient exchanges of one step once a step has run."""

    buckets: list[int] = []
    exchanges = 0

    def run(self, micro) -> torch.Tensor:
        raise NotImplementedError


class TorchStepper(Stepper):
    """Eager torch: the module (plain or wrapped in DDP), ``torch.optim.AdamW``."""

    def __init__(self, module: nn.Module, workload: Workload, loss_fn, lr: float) -> None:
        self.module, self.workload, self.loss_fn = module, workload, loss_fn
        self.inner = module.module if hasattr(module, "no_sync") else module
        self.optimizer = torch.optim.AdamW(module.parameters(), lr=lr,
                                           fused=workload.device.type == "cuda")
        self.buckets, self.exchanges = [], 0

    def hook(self, sync_fn):
        def counted(state, bucket):
            self.exchanges += 1
            self._seen.append(bucket.buffer().numel() * bucket.buffer().element_size())
            return sync_fn(state, bucket)
        self._seen: list[int] = []
        return counted

    def _loss(self, x, y):
        # DDP hooks fire from the wrapper's forward: call it, then the family's loss on its output
        ctx = (torch.autocast("cuda", dtype=self.workload.autocast)
               if self.workload.autocast is not None else contextlib.nullcontext())
        with ctx:
            if self.module is self.inner:
                return self.loss_fn(self.inner, x, y)
            return self.loss_fn(_Through(self.module), x, y)

    def run(self, micro):
        self.optimizer.zero_grad(set_to_none=True)
        if hasattr(self, "_seen"):
            self._seen.clear()
        total = None
        for i, (x, y) in enumerate(micro):
            last = i == len(micro) - 1
            held = contextlib.nullcontext() if last or self.module is self.inner else self.module.no_sync()
            with held:
                loss = self._loss(x, y)
                loss.backward()
            total = loss.detach() if total is None else total + loss.detach()
        self.optimizer.step()
        if hasattr(self, "_seen") and self._seen:
            self.buckets = list(self._seen)
        return total


class _Through:
    """What ``loss_fn`` sees in place of the model under DDP: ``loss(x, y)`` goes through the
    wrapper's forward (a :class:`LossModule` inside), where DDP arms its gradient hooks."""

    def __init__(self, wrapper) -> None:
        self._wrapper = wrapper

    def loss(self, x, y):
        return self._wrapper(x, y)


class LossModule(nn.Module):
    """``forward(x, y) -> loss`` so that DDP's forward hooks see the whole computation."""

    def __init__(self, model: nn.Module) -> None:
        super().__init__()
        self.model = model

    def forward(self, x, y):
        return self.model.loss(x, y)


class FlatStepper(Stepper):
    """The flat-buffer trainer of this library (CUDA-graph replay when it can)."""

    def __init__(self, model, workload: Workload, loss_fn, lr: float, topology, graph: bool,
                 bucket_mb: float, weighted: bool) -> None:
        from gpubridge_b200.parallel.trainer import DataParallelTrainer
        self.trainer = DataParallelTrainer(model, loss_fn, topology=topology, lr=lr,
                                           autocast=workload.autocast, bucket_mb=bucket_mb,
                                           graph=graph, unit_grad=not weighted,
                                           exchange=topology is not None)
        self.buckets = [(hi - lo) * 4 for lo, hi, _ in self.trainer._buckets] if self.trainer.world > 1 else []
        self.exchanges = 0

    def run(self, micro):
        self.exchanges += len(self.buckets)
        if len(micro) == 1:
            return self.trainer.step(*micro[0])
        return self.trainer.step_accumulated(micro)


# -- timing ----------------------------------------------------------------------------------------
def timed(device: torch.device, fn) -> float:
    """Seconds of ``fn()`` with the device idle before and after (CUDA events on a GPU)."""
    sync(device)
    if device.type == "cuda":
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        fn()
        stop.record()
        stop.synchronize()
        return start.elapsed_time(stop) / 1e3
    t0 = time.perf_counter()
    fn()
    return time.perf_counter() - t0


def run_phase(stepper: Stepper, data, sizes, device, warmup: int, steps: int) -> tuple[list[float], list[float]]:
    times, losses = [], []
    for i in range(warmup + steps):
        x, y = data[i % len(data)]
        micro = list(zip(x.split(sizes), y.split(sizes)))
        box = []
        t = timed(device, lambda: box.append(stepper.run(micro)))
        if i >= warmup:
            times.append(t)
        losses.append(float(box[0]))
    return times, losses


def memory(device: torch.device) -> dict | None:
    if device.type != "cuda":
        return None
    stats = torch.cuda.memory_stats(device)
    out = {"max_allocated_mib": round(torch.cuda.max_memory_allocated(device) / 2**20, 1),
           "max_reserved_mib": round(torch.cuda.max_memory_reserved(device) / 2**20, 1),
           "num_alloc_retries": stats.get("num_alloc_retries", 0),
           "total_mib": round(torch.cuda.get_device_properties(device).total_memory / 2**20, 1)}
    torch.cuda.reset_peak_memory_stats(device)
    return out


def gather(value):
    out = [None] * dist.get_world_size()
    dist.all_gather_object(out, value)
    return out


def ms(seconds: float) -> float:
    return round(seconds * 1e3, 3)


# -- main ------------------------------------------------------------------------------------------
def parse(argv=None) -> argparse.Namespace:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", choices=sorted(WORKLOADS), default="gpt2-small")
    sizes = ap.add_mutually_exclusive_group()
    sizes.add_argument("--batch-size", type=int, help="samples per rank and step")
    sizes.add_argument("--batch-sizes", help="one batch per rank, comma-separated, in rank order")
    sizes.add_argument("--global-batch", type=int, help="samples per step over all ranks")
    ap.add_argument("--balance", action="store_true", help="split --global-batch by measured speed")
    ap.add_argument("--calibration-batch", type=int)
    ap.add_argument("--calibration-steps", type=int, default=3)
    ap.add_argument("--accumulate", type=int, default=1, metavar="K")
    ap.add_argument("--seq-len", type=int, help="GPT models only")
    ap.add_argument("--steps", type=int, default=10, help="timed steps per phase")
    ap.add_argument("--warmup-steps", type=int, default=3)
    ap.add_argument("--comm-trials", type=int, default=5)
    ap.add_argument("--bucket-mb", type=float, default=25.0)
    ap.add_argument("--lr", type=float, default=1e-4)
    ap.add_argument("--controlled", action="store_true")
    ap.add_argument("--engine", choices=("ddp", "trainer"), default=None,
                    help="default: trainer on GPUs, ddp on CPU ranks")
    ap.add_argument("--no-graph", action="store_true", help="trainer engine: run the step eagerly")
    ap.add_argument("--grad-sync", choices=("gpubridge", "native"), default="gpubridge")
    ap.add_argument("--bridge", default=os.environ.get("GPUBRIDGE_BRIDGE", "").strip() or None)
    ap.add_argument("--timeout", type=float, default=float(os.environ.get("KIT_TIMEOUT", "600")))
    ap.add_argument("--json", type=Path)
    args = ap.parse_args(argv)
    if args.balance and args.global_batch is None:
        ap.error("--balance needs --global-batch")
    if args.controlled and args.balance:
        ap.error("--controlled keeps fixed batches: not with --balance")
    if args.accumulate < 1:
        ap.error("--accumulate must be at least 1")
    if args.grad_sync == "native" and args.engine == "trainer":
        ap.error("--grad-sync native is plain DistributedDataParallel: use --engine ddp")
    return args


def main(argv=None) -> int:
    args = parse(argv)
    topology = gb.init(timeout=timedelta(seconds=args.timeout), **({"bridge": args.bridge} if args.bridge else {}))
    rank, world, device = topology.rank, topology.world_size, topology.device
    engine = args.engine or ("trainer" if device.type == "cuda" and args.grad_sync == "gpubridge" else "ddp")
    if device.type == "cpu":
        torch.set_num_threads(1)
    if args.controlled:
        torch.use_deterministic_algorithms(True, warn_only=True)
        torch.backends.cuda.matmul.allow_tf32 = False
        torch.backends.cudnn.allow_tf32 = False
        os.environ.setdefault("CUBLAS_WORKSPACE_CONFIG", ":4096:8")
    if args.grad_sync == "native" and len({p.vendor for p in topology.peers}) > 1:
        raise SystemExit("--grad-sync native: one vendor's library cannot span a mixed-vendor run")
    workload = Workload(args.model, args.seq_len, device, args.controlled)
    k = args.accumulate

    # -- each rank's batch ------------------------------------------------------------------------
    calibration = None
    if args.batch_sizes:
        shares = [int(v) for v in args.batch_sizes.split(",")]
        if len(shares) != world or min(shares) < k:
            raise SystemExit(f"--batch-sizes needs {world} values of at least {k}")
        split = "given"
    elif args.global_batch is not None and args.balance:
        trial = args.calibration_batch or max(1, args.global_batch // world)
        trial_sizes = cut(max(trial, k), k)
        probe = TorchStepper(workload.build(), workload, workload.loss_fn(None), args.lr)
        times, _ = run_phase(probe, workload.data(sum(trial_sizes), rank), trial_sizes, device, 1,
                             args.calibration_steps)
        per_sample = statistics.median(times) / sum(trial_sizes)
        everyone = gather(per_sample)
        shares = speed_shares(args.global_batch, everyone, floor=k)
        calibration = {"batch": sum(trial_sizes), "steps": args.calibration_steps,
                       "seconds_per_sample": everyone}
        del probe
        split = "balanced"
    elif args.global_batch is not None:
        shares = even_shares(args.global_batch, world)
        if min(shares) < k:
            raise SystemExit(f"--global-batch {args.global_batch} leaves a rank fewer than {k} samples")
        split = "even"
    else:
        shares = [args.batch_size or workload.default_batch] * world
        split = "equal"
    batch, total = shares[rank], sum(shares)
    sizes = cut(batch, k)
    weighted = len(set(shares)) > 1 or k > 1
    weight = world / total if weighted else None
    loss_fn = workload.loss_fn(weight)
    data = workload.data(batch, rank)
    inputs_digest = digest([t.float() for pair in data for t in pair]) if args.controlled else None

    # -- phase 1: compute alone --------------------------------------------------------------------
    model = workload.build()
    seeded = digest(model.parameters()) if args.controlled else None
    if device.type == "cuda":
        torch.cuda.reset_peak_memory_stats(device)
    graph = engine == "trainer" and not args.no_graph and k == 1
    if engine == "trainer":
        alone: Stepper = FlatStepper(model, workload, loss_fn, args.lr, None, graph, args.bucket_mb, weighted)
    else:
        alone = TorchStepper(model, workload, loss_fn, args.lr)
    compute, _ = run_phase(alone, data, sizes, device, args.warmup_steps, args.steps)
    mem = {"compute": memory(device)}
    del alone
    if args.controlled:
        model = workload.build()

    # -- phase 2: with the exchange ----------------------------------------------------------------
    native_group = None
    if engine == "trainer":
        together: Stepper = FlatStepper(model, workload, loss_fn, args.lr, topology, graph,
                                        args.bucket_mb, weighted)
        if world > 1:
            gb.broadcast(together.trainer.flat_param, 0)
    else:
        wrapped = LossModule(model)
        if args.grad_sync == "native":
            native_group = dist.new_group(backend="nccl" if device.type == "cuda" else "gloo",
                                          timeout=timedelta(seconds=args.timeout))
        ddp = nn.parallel.DistributedDataParallel(
            wrapped, device_ids=[device.index] if device.type == "cuda" else None,
            process_group=native_group, bucket_cap_mb=args.bucket_mb, broadcast_buffers=False,
            gradient_as_bucket_view=True)
        together = TorchStepper(ddp, workload, loss_fn, args.lr)
        if args.grad_sync == "gpubridge":
            ddp.register_comm_hook(None, together.hook(gb.ddp_comm_hook))
        else:
            from torch.distributed.algorithms.ddp_comm_hooks.default_hooks import allreduce_hook
            ddp.register_comm_hook(native_group, together.hook(allreduce_hook))
    if args.controlled and digest(model.parameters()) != seeded:
        raise RuntimeError("controlled run: the parameters before the ddp phase differ from the seeded model")
    step_times, losses = run_phase(together, data, sizes, device, args.warmup_steps, args.steps)
    mem["ddp"] = memory(device)
    if engine == "trainer":
        together.trainer.check()

    params = [p.detach() for p in model.parameters()]
    finite = all(bool(torch.isfinite(p).all()) for p in params)
    mine = (digest(params), float(sum(p.double().sum() for p in params)))
    everyone_params = gather(mine)

    # -- phase 3: the exchanges alone ---------------------------------------------------------------
    buckets = list(together.buckets)
    exchanges_per_step = together.exchanges / (args.warmup_steps + args.steps)
    tensors = [torch.zeros(max(1, b // 4), dtype=torch.float32, device=device) for b in buckets]

    def exchange_all():
        if args.grad_sync == "native":
            works = [dist.all_reduce(t, group=native_group, async_op=True) for t in tensors]
        else:
            works = [gb.all_reduce(t, gb.ReduceOp.AVG, async_op=True) for t in tensors]
        for w in works:
            w.wait()

    comm = []
    if world > 1 and tensors:
        for i in range(2 + args.comm_trials):
            t = timed(device, exchange_all)
            if i >= 2:
                comm.append(t)
    mem["comm_alone"] = memory(device)

    # -- the record -------------------------------------------------------------------------------
    per_rank = gather({"compute": statistics.median(compute), "steps": step_times, "batch": batch,
                       "micro": sizes, "comm": statistics.median(comm) if comm else 0.0,
                       "memory": mem if device.type == "cuda" else None})
    slowest_compute = max(r["compute"] for r in per_rank)
    ddp_step = statistics.median(max(r["steps"][i] for r in per_rank) for i in range(args.steps))
    comm_alone = max(r["comm"] for r in per_rank)
    exposed = ddp_step - slowest_compute
    record = {
        "model": args.model, "engine": engine, "grad_sync": args.grad_sync, "world_size": world,
        "cuda_graph": graph, "dtype": "bf16 autocast" if workload.autocast is not None else "fp32",
        "seq_len": workload.seq, "global_batch": total, "split": split, "accumulate": k,
        "ddp_step_ms": ms(ddp_step), "slowest_compute_ms": ms(slowest_compute),
        "exposed_comm_ms": ms(exposed), "comm_alone_ms": ms(comm_alone),
        "hidden_comm_ms": ms(max(0.0, comm_alone - max(0.0, exposed))),
        "samples_per_s": round(total / ddp_step, 2),
        "tokens_per_s": round(total * workload.seq / ddp_step, 1) if workload.seq else None,
        "bucket_bytes": buckets, "exchanges_per_step": exchanges_per_step,
        "exchanges_per_sample": exchanges_per_step / total,
        "ranks": [{"rank": r, "batch": v["batch"], "micro_batches": v["micro"],
                   "compute_ms": ms(v["compute"]), "per_sample_compute_ms": ms(v["compute"] / v["batch"]),
                   "waiting_ms": ms(slowest_compute - v["compute"]),
                   "alone_samples_per_s": round(v["batch"] / v["compute"], 2), "memory": v["memory"]}
                  for r, v in enumerate(per_rank)],
        "calibration": calibration, "loss_first": losses[0], "loss_last": losses[-1],
        "params_identical": len({d for d, _ in everyone_params}) == 1,
        "params_sum_spread": max(s for _, s in everyone_params) - min(s for _, s in everyone_params),
        "params_finite": finite,
        "controlled": {"inputs": inputs_digest, "initial_parameters": seeded} if args.controlled else None,
        "note": ("CPU/Gloo stand-in, not an NCCL result" if args.grad_sync == "native" and device.type == "cpu"
                 else None),
        "run": run_info(topology), "environment": environment(),
    }
    if rank == 0:
        print(f"{args.model} on {world} ranks ({engine}, {args.grad_sync}): {record['samples_per_s']} samples/s; "
              f"step {record['ddp_step_ms']} ms = compute {record['slowest_compute_ms']} + exposed exchange "
              f"{record['exposed_comm_ms']} (alone {record['comm_alone_ms']}, hidden {record['hidden_comm_ms']}); "
              f"parameters {'identical' if record['params_identical'] else 'DIFFER'}")
        if args.json:
            write_json(args.json, record)
    all_finite = all(gather(finite))
    if native_group is not None:
        dist.destroy_process_group(native_group)
    gb.destroy()
    return 0 if all_finite else 1


if __name__ == "__main__":
    sys.exit(main())
