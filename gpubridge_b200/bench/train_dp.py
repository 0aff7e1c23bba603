"""Data-parallel training throughput of the Llama-style models through backend="gpubridge":
``ddp``, ``fsdp2`` (``fully_shard`` on a 1-D mesh), ``hsdp`` (shard inside an island,
replicate across islands; the cross-island gradient all-reduce is the compressed one when
``GPUBRIDGE_BRIDGE_COMPRESSION`` is set) and ``fused`` (recorded runs: this library's own
sharding - every block's Linear layers become ``ShardedLinear``, whose all-gather is fused
into the tcgen05 GEMM; the rest stays replicated and is averaged with one all-reduce).  Counterpart of the reference's
scripts/gpu/train_dp.py.

    GPUBRIDGE_ISLANDS=4,4 GPUBRIDGE_BRIDGE_COMPRESSION=fp8 GPUBRIDGE_CODEC_FORMAT=b200 \
      python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 \
      -m gpubridge_b200.bench.train_dp --model llama3-8b --mode hsdp --batch 1 --seq 4096

Timing: warm-up steps, then ``--steps`` steps between CUDA events with a barrier and a
synchronize on both sides; the slowest rank counts.  One JSON line on rank 0.

With ``--json PATH`` the run is a *recorded* one instead (what ``kit.report dp`` lays side by
side): every step trains on ``llama.rule_batch(step)`` - the same ``--global-batch`` rows for
any world size, learnable, so loss curves of different runs can be compared - and each rank
takes a contiguous share of the rows: equal shares, ``--shares speed`` (proportional to each
rank's measured step rate) or ``--shares 5,3``.  A rank's loss is weighted by
world x share / global batch, so the average every mode takes is the mean gradient of the
whole batch.  ``--mode single`` is the one-GPU baseline on the whole batch (``--micro`` rows
at a time, gradients accumulated).  Recorded: every step's loss over the whole batch and its
time (each step synchronised, the loss gathered outside the timed part); every
``--check-every`` steps whether the replicas hold the same parameter bits (``ddp``: all
ranks; ``hsdp``: the replicate groups; ``fsdp2``: nothing to compare) and the spread of
their parameter sums; tokens/s from the median step after the warm-up.
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


def shares_for(weights: list[float], total: int) -> list[int]:
    """``total`` rows in proportion to ``weights``, at least one each: floors first, then the
    largest remainders (the lower rank on a tie)."""
    world = len(weights)
    if total < world:
        raise ValueError(f"{total} rows cannot give each of {world} ranks one")
    scale = (total - world) / sum(weights)
    exact = [w * scale for w in weights]
    shares = [1 + int(e) for e in exact]
    order = sorted(range(world), key=lambda r: (-(exact[r] - int(exact[r])), r))
    for r in order[:total - sum(shares)]:
        shares[r] += 1
    return shares


def _digest(tensors) -> tuple[str, float]:
    import hashlib
    h, total = hashlib.sha256(), 0.0
    for t in tensors:
        local = t.detach()
        local = local.to_local() if hasattr(local, "to_local") else local
        h.update(local.float().cpu().numpy().tobytes())
        total += float(local.double().sum())
    return h.hexdigest()[:16], total


def recorded(args) -> int:
    """The ``--json`` run: same data at any scale, weighted shares, per-step record."""
    import statistics
    from pathlib import Path

    from gpubridge_b200.kit import environment, write_json
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    on_gpu = torch.cuda.is_available() and not os.environ.get("GPUBRIDGE_VENDOR")
    device = torch.device("cuda", local) if on_gpu else torch.device("cpu")
    if on_gpu:
        torch.cuda.set_device(device)
    else:
        torch.set_num_threads(1)
    single = args.mode == "single"
    if single and world != 1:
        raise SystemExit("--mode single is one process")
    if not single:
        with warnings.catch_warnings():
            warnings.simplefilter("ignore", gb.SplitTestWarning)
            dist.init_process_group(args.backend if on_gpu or args.backend == "gpubridge" else "gloo")
    dtype = torch.bfloat16 if on_gpu else torch.float32
    model = llama.build(args.model, seed=0, device=device, dtype=torch.float32, rng=args.rng)
    config = model.config
    total = args.global_batch or args.batch * world
    replicas = None                       # process group whose members hold the same parameters
    if args.mode == "ddp":
        from torch.nn.parallel import DistributedDataParallel as DDP
        model = DDP(model, device_ids=[local] if on_gpu else None)
        replicas = dist.group.WORLD
    elif args.mode == "fused":
        from gpubridge_b200.parallel.sharded_model import ReplicatedSync, shard_linears
        if args.backend != "gpubridge":
            raise SystemExit("--mode fused runs on the gpubridge backend")
        if on_gpu:
            model.to(dtype)                      # the fused GEMM takes bf16 operands
        topology = gb.get_topology()
        sharded = shard_linears(model.blocks, topology)
        replicated = ReplicatedSync(model, topology)
        replicas = dist.group.WORLD             # the parameters that stayed whole must stay identical
    elif args.mode in ("fsdp2", "hsdp"):
        from torch.distributed.device_mesh import init_device_mesh
        from torch.distributed.fsdp import MixedPrecisionPolicy, fully_shard
        kind = "cuda" if on_gpu else "cpu"
        if args.mode == "hsdp":
            islands = [int(v) for v in os.environ.get("GPUBRIDGE_ISLANDS", "").split(",") if v]
            shard = islands[0] if islands else max(1, world // 2)
            mesh = init_device_mesh(kind, (world // shard, shard), mesh_dim_names=("replicate", "shard"))
            replicas = mesh.get_group("replicate")
        else:
            mesh = init_device_mesh(kind, (world,))
        policy = MixedPrecisionPolicy(param_dtype=dtype, reduce_dtype=dtype) if on_gpu else MixedPrecisionPolicy()
        for block in model.blocks:
            fully_shard(block, mesh=mesh, mp_policy=policy)
        fully_shard(model, mesh=mesh, mp_policy=policy)
    optimizer = torch.optim.AdamW(model.parameters(), lr=args.lr, fused=on_gpu)
    core = model.module if hasattr(model, "module") else model

    def forward_loss(x, y):
        if args.mode in ("single", "ddp") and on_gpu:
            with torch.autocast("cuda", dtype=dtype):
                logits = model(x)
        else:
            logits = model(x)
        return torch.nn.functional.cross_entropy(logits.view(-1, logits.shape[-1]).float(), y.reshape(-1))

    def everyone(value):
        if single:
            return [value]
        out = [None] * world
        dist.all_gather_object(out, value)
        return out

    def wait():
        if on_gpu:
            torch.cuda.synchronize(device)

    # -- shares ------------------------------------------------------------------------------------
    calibration = None
    if single or args.shares == "equal":
        shares = shares_for([1.0] * world, total)
    elif args.shares == "speed":
        rows = max(1, total // world)
        x, y = (t.to(device) for t in llama.rule_batch(config, 0, rows, args.seq, seed=99))
        took = []
        for i in range(4):           # lr is untouched: these steps use a throw-away optimizer state
            wait()
            t0 = time.perf_counter()
            forward_loss(x, y).backward()
            wait()
            if i:
                took.append(time.perf_counter() - t0)
            model.zero_grad(set_to_none=True)
        mine = rows / statistics.median(took)
        calibration = {"rows": rows, "rows_per_s": everyone(mine)}
        shares = shares_for(calibration["rows_per_s"], total)
    else:
        shares = [int(v) for v in args.shares.split(",")]
        if len(shares) != world or sum(shares) != total or min(shares) < 1:
            raise SystemExit(f"--shares needs {world} positive row counts that add up to {total}")
    lo = sum(shares[:rank])
    mine = shares[rank]
    weight = world * mine / total
    micro = args.micro if single and args.micro else mine

    losses, times, checks = [], [], []
    for step in range(args.warmup + args.steps):
        x, y = llama.rule_batch(config, step, total, args.seq)
        x, y = x[lo:lo + mine].to(device), y[lo:lo + mine].to(device)
        wait()
        if not single:
            dist.barrier()
        t0 = time.perf_counter()
        optimizer.zero_grad(set_to_none=True)
        local_loss = 0.0
        for start in range(0, mine, micro):
            part = slice(start, min(mine, start + micro))
            rows = part.stop - part.start
            loss = forward_loss(x[part], y[part]) * (weight * rows / mine)
            loss.backward()
            local_loss += float(loss.detach()) if not on_gpu else loss.detach()
        if args.mode == "fused":
            replicated.average_gradients()
        optimizer.step()
        wait()
        times.append(max(everyone(time.perf_counter() - t0)))
        # the weighted losses average to the whole batch's mean loss
        losses.append(sum(float(v) for v in everyone(float(local_loss))) / world)
        if replicas is not None and args.check_every and (step + 1) % args.check_every == 0:
            got = everyone(_digest(replicated.params if args.mode == "fused" else core.parameters()))
            members = dist.get_process_group_ranks(replicas)
            mates = everyone(members)
            groups = {tuple(m) for m in mates}
            same = all(len({got[r][0] for r in g}) == 1 for g in groups)
            spread = max(max(got[r][1] for r in g) - min(got[r][1] for r in g) for g in groups)
            checks.append({"step": step, "identical": same, "sum_spread": spread})
    timed = times[args.warmup:] or times
    median = statistics.median(timed)
    record = {"bench": "train_dp", "recorded": True, "model": args.model, "mode": args.mode,
              "backend": args.backend if not single else None, "world": world, "global_batch": total,
              "seq": args.seq, "shares": shares, "calibration": calibration,
              "compression": os.environ.get("GPUBRIDGE_BRIDGE_COMPRESSION", ""),
              "losses": losses, "step_ms": [round(t * 1e3, 3) for t in times],
              "median_step_ms": round(median * 1e3, 3),
              "tokens_per_s": round(total * args.seq / median, 1), "warmup_steps": args.warmup,
              "parameter_checks": checks,
              "parameters_identical": all(c["identical"] for c in checks) if checks else None,
              "parameters": sum(p.numel() for p in core.parameters()), "environment": environment()}
    if args.mode == "fused":
        record["sharded_layers"] = len(sharded)
        record["parameter_bytes"] = replicated.memory(model)
    if rank == 0:
        print(json.dumps({k: v for k, v in record.items() if k not in ("losses", "step_ms", "environment",
                                                                         "parameter_checks")}), flush=True)
        write_json(Path(args.json), record)
    if not single:
        dist.destroy_process_group()
    return 0 if record["parameters_identical"] in (True, None) else 1


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--model", default="llama-125m", choices=sorted(llama.CONFIGS))
    ap.add_argument("--mode", default="fsdp2", choices=("single", "ddp", "fsdp2", "hsdp", "fused"))
    ap.add_argument("--batch", type=int, default=4)
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--lr", type=float, default=3e-4)
    ap.add_argument("--backend", default="gpubridge", help="gpubridge or nccl (the baseline)")
    ap.add_argument("--rng", default="device", choices=("cpu", "device"),
                    help="where the random initial weights are drawn (same seed on every rank)")
    ap.add_argument("--json", help="recorded run: rank 0 writes the record here")
    ap.add_argument("--global-batch", type=int, help="recorded run: rows per step over all ranks "
                    "(default --batch x world)")
    ap.add_argument("--shares", default="equal", help="recorded run: equal, speed, or rows per rank a,b,...")
    ap.add_argument("--micro", type=int, help="--mode single: rows per micro-batch")
    ap.add_argument("--check-every", type=int, default=10)
    args = ap.parse_args(argv)
    if args.json:
        return recorded(args)

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
    elif args.mode == "fused":
        from gpubridge_b200.parallel.sharded_model import ReplicatedSync, shard_linears
        if args.backend != "gpubridge":
            raise SystemExit("--mode fused runs on the gpubridge backend")
        if on_gpu:
            model.to(dtype)                      # the fused GEMM takes bf16 operands
        shard_linears(model.blocks, gb.get_topology())
        replicated = ReplicatedSync(model, gb.get_topology())
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
        if args.mode == "fused":
            replicated.average_gradients()
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
    front_end = _front_end_calls(device, locals().get("mesh"))
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
            "clocks": clocks, "front_end": front_end,
        }), flush=True)
    dist.destroy_process_group()
    return 0


def _front_end_calls(device, mesh) -> dict | None:
    """How many collective calls the C++ front end launched itself and how many it handed to
    the Python group, summed over the world group and the mesh's groups (None when another
    backend, or the Python group, answers)."""
    groups = [dist.group.WORLD]
    if mesh is not None:
        try:
            groups += list(mesh.get_all_groups())
        except Exception:  # noqa: BLE001 - a mesh without groups of its own
            pass
    native = fallback = 0
    seen = False
    for group in groups:
        try:
            backend = group._get_backend(device)
        except Exception:  # noqa: BLE001
            continue
        if hasattr(backend, "native_calls"):
            seen = True
            native += int(backend.native_calls)
            fallback += int(backend.fallback_calls)
    return {"native_calls": native, "fallback_calls": fallback} if seen else None


if __name__ == "__main__":
    sys.exit(main())
