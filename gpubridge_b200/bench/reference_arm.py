"""The reference build measured beside this one, on the same box, with the same method.

Run it BY PATH (never with ``-m``: that would import this package first)::

    GPUBRIDGE_SPLIT_TEST=half python -m torch.distributed.run --nproc-per-node 8 \
        --master-addr 127.0.0.1 gpubridge_b200/bench/reference_arm.py sweep --largest 64M
    ... reference_arm.py p2p --largest 64M
    ... reference_arm.py train --model llama-1.3b --mode fsdp2 --batch 4 --seq 2048

Everything imported here is the unmodified reference package installed under
``baseline/_ref`` (its own NCCL islands joined by its default Gloo bridge, its policies, its
``backend="gpubridge"``), PyTorch, and the standard library: no module, model or kernel of
``gpubridge_b200`` is on this path.  The models for ``train`` are therefore written out below
in stock PyTorch modules (the shapes of the benchmark configurations).

Timing is this repository's method for every arm (the reference's own,
scripts/gpu/bench_all_reduce.py:125-197): warm-ups, then trials bracketed by CUDA events on
the current stream, a trial's latency is the slowest rank's, the median over trials is
reported; ``busbw = algbw * 2 (n-1) / n`` for all_reduce.  Rank 0 prints one JSON line per
row; when the reference cannot be imported it prints ``{"impl": "reference", "unavailable":
...}`` and exits 0.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import time
import warnings

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
REF = os.path.join(ROOT, "baseline", "_ref")

BUS = {"all_reduce": lambda n: 2 * (n - 1) / n, "all_gather": lambda n: (n - 1) / n,
       "reduce_scatter": lambda n: (n - 1) / n, "broadcast": lambda n: 1.0}
UNITS = {"K": 1 << 10, "M": 1 << 20, "G": 1 << 30}


def parse_size(text: str) -> int:
    text = text.strip().upper().rstrip("B")
    if text and text[-1] in UNITS:
        return int(float(text[:-1]) * UNITS[text[-1]])
    return int(text)


def load_reference():
    """The reference package, or the reason it cannot be had."""
    if not os.path.isdir(os.path.join(REF, "gpubridge")):
        return None, "baseline/_ref is not installed"
    sys.path[:] = [p for p in sys.path if os.path.abspath(p or ".") != ROOT]      # never this package
    sys.path.insert(0, REF)
    try:
        import gpubridge
    except Exception as failure:  # noqa: BLE001
        return None, f"import gpubridge failed: {failure}"[:200]
    return gpubridge, ""


def rank_info() -> tuple[int, int, int]:
    return (int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0")),
            int(os.environ.get("WORLD_SIZE", "1")))


def emit(row: dict) -> None:
    if rank_info()[0] == 0:
        print(json.dumps(row), flush=True)


def slowest_rank_median(gpubridge, call, device, trials: int, seconds: float, warmup: int = 5) -> float:
    import torch
    for _ in range(warmup):
        call()
    torch.cuda.synchronize(device)
    gpubridge.barrier()
    samples, began = [], time.monotonic()
    for _ in range(trials):
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        call()
        end.record()
        end.synchronize()
        worst = torch.tensor([start.elapsed_time(end), float(time.monotonic() - began > seconds)],
                             dtype=torch.float64, device=device)
        gpubridge.all_reduce(worst, gpubridge.ReduceOp.MAX)
        samples.append(float(worst[0]))
        if float(worst[1]) > 0:
            break
    return statistics.median(samples)


# ---- collectives ----------------------------------------------------------------------------------------
def sweep(args) -> int:
    gpubridge, why = load_reference()
    if gpubridge is None:
        emit({"impl": "reference", "unavailable": why})
        return 0
    import torch
    rank, local, world = rank_info()
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        topology = gpubridge.init(**({"policy": args.policy} if args.policy else {}))
    try:
        for op in args.ops.split(","):
            for dtype_name in args.dtypes.split(","):
                dtype = getattr(torch, dtype_name)
                esize = torch.empty(0, dtype=dtype).element_size()
                size = parse_size(args.smallest)
                while size <= parse_size(args.largest):
                    n = max(world, size // esize // world * world)
                    full = torch.randn(n, generator=torch.Generator().manual_seed(1234 + rank)).to(dtype).to(device)
                    moved = n * esize
                    if op == "all_reduce":
                        call = lambda: gpubridge.all_reduce(full)                       # noqa: E731
                    elif op == "broadcast":
                        call = lambda: gpubridge.broadcast(full, 0)                     # noqa: E731
                    elif op == "all_gather":
                        part = full[: n // world]
                        out = torch.empty(n, dtype=dtype, device=device)
                        call = lambda: gpubridge.all_gather_into_tensor(out, part)      # noqa: E731
                    else:
                        out = torch.empty(n // world, dtype=dtype, device=device)
                        call = lambda: gpubridge.reduce_scatter_tensor(out, full)       # noqa: E731
                    ms = slowest_rank_median(gpubridge, call, device, args.trials, args.seconds)
                    algbw = moved / (ms * 1e-3) / 1e9
                    emit({"impl": "reference", "op": op, "dtype": dtype_name, "bytes": moved,
                          "target": "reference", "ms": round(ms, 5), "algbw_gbs": round(algbw, 3),
                          "busbw_gbs": round(algbw * BUS[op](world), 3), "world": world,
                          "islands": [len(i.ranks) for i in topology.layout.islands],
                          "policy": topology.policy_name,
                          "bridge": getattr(topology.transport, "name", None),
                          "compression": os.environ.get("GPUBRIDGE_BRIDGE_COMPRESSION", "")})
                    size *= 2
    finally:
        gpubridge.destroy()
    return 0


# ---- point to point ----------------------------------------------------------------------------------------
def p2p(args) -> int:
    gpubridge, why = load_reference()
    if gpubridge is None:
        emit({"impl": "reference", "unavailable": why})
        return 0
    import torch
    import torch.distributed as dist
    rank, local, world = rank_info()
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        dist.init_process_group(backend="gpubridge")
        dist.barrier()
    peer = world - 1 - rank                       # pairs across the halves: cross-island when split
    try:
        size = parse_size(args.smallest)
        while size <= parse_size(args.largest):
            send = torch.ones(size, dtype=torch.uint8, device=device)
            recv = torch.empty(size, dtype=torch.uint8, device=device)

            def exchange():
                ops = [dist.P2POp(dist.isend, send, peer), dist.P2POp(dist.irecv, recv, peer)]
                if rank > peer:
                    ops.reverse()
                for work in dist.batch_isend_irecv(ops):
                    work.wait()

            for _ in range(3):
                exchange()
            torch.cuda.synchronize(device)
            dist.barrier()
            samples = []
            for _ in range(args.trials):
                start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                start.record()
                exchange()
                end.record()
                end.synchronize()
                worst = torch.tensor([start.elapsed_time(end)], dtype=torch.float64, device=device)
                dist.all_reduce(worst, op=dist.ReduceOp.MAX)
                samples.append(float(worst))
            ms = statistics.median(samples)
            emit({"impl": "reference", "op": "batch_isend_irecv", "bytes": size, "target": "reference",
                  "ms": round(ms, 5), "gbs_each_way": round(size / (ms * 1e-3) / 1e9, 3), "world": world})
            size *= 2
    finally:
        dist.destroy_process_group()
    return 0


# ---- training through the reference's backend ---------------------------------------------------------------
SHAPES = {   # layers, width, heads, kv heads, ffn, vocabulary, rope base
    "llama-125m": (12, 768, 12, 12, 2048, 32000, 10000.0),
    "llama-1.3b": (24, 2048, 16, 16, 5632, 32000, 10000.0),
    "llama3-8b": (32, 4096, 32, 8, 14336, 128256, 500000.0),
}


def stock_llama(name: str, device, seq: int):
    """The benchmark decoder in stock PyTorch modules: RMSNorm, rotary positions, grouped-query
    attention through ``scaled_dot_product_attention``, SwiGLU; weights N(0, 0.02)."""
    import torch
    import torch.nn as nn
    import torch.nn.functional as F
    layers, width, heads, kv_heads, ffn, vocab, base = SHAPES[name]
    head_dim = width // heads

    class Block(nn.Module):
        def __init__(self):
            super().__init__()
            self.norm1, self.norm2 = nn.RMSNorm(width, eps=1e-5), nn.RMSNorm(width, eps=1e-5)
            self.q = nn.Linear(width, width, bias=False)
            self.kv = nn.Linear(width, 2 * kv_heads * head_dim, bias=False)
            self.o = nn.Linear(width, width, bias=False)
            self.gate_up = nn.Linear(width, 2 * ffn, bias=False)
            self.down = nn.Linear(ffn, width, bias=False)

        def forward(self, x, cos, sin):
            b, t, _ = x.shape
            h = self.norm1(x)
            q = self.q(h).view(b, t, heads, head_dim).transpose(1, 2)
            k, v = self.kv(h).view(b, t, 2, kv_heads, head_dim).unbind(2)
            k, v = k.transpose(1, 2), v.transpose(1, 2)

            def rotate(z):
                a, c = z[..., ::2], z[..., 1::2]
                return torch.stack((a * cos - c * sin, a * sin + c * cos), dim=-1).flatten(-2).to(z.dtype)

            q, k = rotate(q), rotate(k)
            y = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=kv_heads != heads)
            x = x + self.o(y.transpose(1, 2).reshape(b, t, width))
            gate, up = self.gate_up(self.norm2(x)).chunk(2, dim=-1)
            return x + self.down(F.silu(gate) * up)

    class Decoder(nn.Module):
        def __init__(self):
            super().__init__()
            self.embed = nn.Embedding(vocab, width)
            self.blocks = nn.ModuleList(Block() for _ in range(layers))
            self.norm = nn.RMSNorm(width, eps=1e-5)
            self.head = nn.Linear(width, vocab, bias=False)
            inv = 1.0 / base ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim)
            angle = torch.outer(torch.arange(seq, dtype=torch.float32), inv)
            self.register_buffer("cos", angle.cos(), persistent=False)
            self.register_buffer("sin", angle.sin(), persistent=False)

        def forward(self, tokens):
            x = self.embed(tokens)
            for block in self.blocks:
                x = block(x, self.cos[: tokens.shape[1]], self.sin[: tokens.shape[1]])
            return self.head(self.norm(x))

    torch.manual_seed(0)
    with torch.device(device):
        model = Decoder()
    for module in model.modules():
        if isinstance(module, (nn.Linear, nn.Embedding)):
            nn.init.normal_(module.weight, mean=0.0, std=0.02)
    return model, vocab


def train(args) -> int:
    gpubridge, why = load_reference()
    if gpubridge is None:
        emit({"impl": "reference", "unavailable": why})
        return 0
    import torch
    import torch.distributed as dist
    import torch.nn.functional as F
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.fsdp import MixedPrecisionPolicy, fully_shard
    rank, local, world = rank_info()
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    try:
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            dist.init_process_group(backend="gpubridge")
            dist.barrier()
        model, vocab = stock_llama(args.model, device, args.seq)
        if args.mode == "hsdp":
            shard = max(1, world // args.islands)
            mesh = init_device_mesh("cuda", (world // shard, shard), mesh_dim_names=("replicate", "shard"))
        else:
            mesh = init_device_mesh("cuda", (world,))
        policy = MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.bfloat16)
        for block in model.blocks:
            fully_shard(block, mesh=mesh, mp_policy=policy)
        fully_shard(model, mesh=mesh, mp_policy=policy)
        optimizer = torch.optim.AdamW(model.parameters(), lr=3e-4, fused=True)
        tokens = torch.randint(vocab, (args.batch, args.seq + 1), generator=torch.Generator().manual_seed(rank))
        x, y = tokens[:, :-1].contiguous().to(device), tokens[:, 1:].contiguous().to(device)

        def step():
            optimizer.zero_grad(set_to_none=True)
            logits = model(x)
            loss = F.cross_entropy(logits.view(-1, logits.shape[-1]).float(), y.reshape(-1))
            loss.backward()
            optimizer.step()
            return loss.detach()

        for _ in range(args.warmup):
            loss = step()
        torch.cuda.synchronize(device)
        dist.barrier()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(args.steps):
            loss = step()
        end.record()
        torch.cuda.synchronize(device)
        dist.barrier()
        worst = torch.tensor([start.elapsed_time(end)], dtype=torch.float64, device=device)
        dist.all_reduce(worst, op=dist.ReduceOp.MAX)
        total = args.batch * args.seq * world * args.steps
        emit({"impl": "reference", "bench": "train_dp", "model": args.model, "mode": args.mode,
              "backend": "gpubridge (reference build)", "world": world, "batch_per_gpu": args.batch,
              "seq": args.seq, "steps": args.steps, "ms_per_step": round(float(worst) / args.steps, 3),
              "tokens_per_s": round(total / (float(worst) * 1e-3), 1), "loss": round(float(loss), 4),
              "compression": os.environ.get("GPUBRIDGE_BRIDGE_COMPRESSION", "")})
    except Exception as failure:  # noqa: BLE001 - the arm reports, it does not take the job down
        emit({"impl": "reference", "unavailable": f"{type(failure).__name__}: {failure}".replace("\n", " ")[:300]})
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()
    return 0


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(description="The reference build's numbers, same box, same method.")
    commands = parser.add_subparsers(dest="command", required=True)
    s = commands.add_parser("sweep", help="collectives through gpubridge.init() and its policies")
    s.add_argument("--smallest", default="4K")
    s.add_argument("--largest", default="64M")
    s.add_argument("--ops", default="all_reduce")
    s.add_argument("--dtypes", default="float32")
    s.add_argument("--policy", default="")
    s.add_argument("--trials", type=int, default=10)
    s.add_argument("--seconds", type=float, default=10.0)
    p = commands.add_parser("p2p", help="batch_isend_irecv between the halves through its backend")
    p.add_argument("--smallest", default="4K")
    p.add_argument("--largest", default="64M")
    p.add_argument("--trials", type=int, default=10)
    t = commands.add_parser("train", help="FSDP2 / HSDP through its backend")
    t.add_argument("--model", default="llama-1.3b", choices=sorted(SHAPES))
    t.add_argument("--mode", default="fsdp2", choices=("fsdp2", "hsdp"))
    t.add_argument("--islands", type=int, default=2)
    t.add_argument("--batch", type=int, default=4)
    t.add_argument("--seq", type=int, default=2048)
    t.add_argument("--steps", type=int, default=5)
    t.add_argument("--warmup", type=int, default=2)
    args = parser.parse_args(argv)
    if os.environ.get("NCCL_DEBUG", "").upper() in ("", "VERSION"):
        os.environ["NCCL_DEBUG"] = "WARN"
    return {"sweep": sweep, "p2p": p2p, "train": train}[args.command](args)


if __name__ == "__main__":
    sys.exit(main())
