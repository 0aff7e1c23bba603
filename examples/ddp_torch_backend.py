"""Train a tiny GPT-2 with ``DistributedDataParallel`` on ``backend="gpubridge"``.

Everything below the import is what a PyTorch user already writes; the only changes to an
NCCL script are ``import gpubridge_b200`` (which registers the backend) and the backend name.

    torchrun --nproc-per-node 8 examples/ddp_torch_backend.py --steps 30
    # no GPUs: four CPU ranks pretending to be two islands of two
    GPUBRIDGE_VENDOR=nvidia GPUBRIDGE_SPLIT_TEST=half \
        torchrun --nproc-per-node 4 examples/ddp_torch_backend.py

At the end every rank hashes its parameters and the hashes are compared through the backend
itself (``all_gather_object``); the script exits 1 if any replica drifted.
"""
from __future__ import annotations

import argparse
import hashlib
import os
import sys

import torch
import torch.distributed as dist
from torch.nn.parallel import DistributedDataParallel

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))   # run from a checkout
import gpubridge_b200  # noqa: E402,F401 - registers backend="gpubridge"
from gpubridge_b200.models import gpt2  # noqa: E402


def pick_device() -> torch.device:
    simulated = bool(os.environ.get("GPUBRIDGE_VENDOR"))
    if simulated or not torch.cuda.is_available():
        return torch.device("cpu")
    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(device)
    return device


def fingerprint(module: torch.nn.Module) -> str:
    digest = hashlib.sha256()
    for _, value in sorted(module.state_dict().items()):
        digest.update(value.detach().to("cpu", torch.float32).numpy().tobytes())
    return digest.hexdigest()[:16]


def main() -> int:
    parser = argparse.ArgumentParser(description="DDP on backend='gpubridge' with a tiny GPT-2.")
    parser.add_argument("--steps", type=int, default=12)
    parser.add_argument("--batch", type=int, default=4, help="sequences per rank and step")
    parser.add_argument("--seq", type=int, default=64)
    args = parser.parse_args()

    dist.init_process_group(backend="gpubridge")
    rank, world = dist.get_rank(), dist.get_world_size()
    device = pick_device()

    torch.manual_seed(2024)                                  # same weights everywhere
    model = gpt2.build("gpt2-tiny").to(device)
    replica = DistributedDataParallel(model, device_ids=[device.index] if device.type == "cuda" else None)
    optimizer = torch.optim.AdamW(replica.parameters(), lr=3e-3, weight_decay=0.0)

    # a fixed set of sequences, dealt out by rank: the loss should fall as they are memorised
    tokens = torch.Generator().manual_seed(7)
    vocab = model.config.vocab
    corpus = torch.randint(0, vocab, (world * args.batch, args.seq + 1), generator=tokens)
    mine = corpus[rank * args.batch:(rank + 1) * args.batch].to(device)
    inputs, targets = mine[:, :-1].contiguous(), mine[:, 1:].contiguous()

    history = []
    for _ in range(args.steps):
        optimizer.zero_grad(set_to_none=True)
        logits = replica(inputs)                             # through DDP: hooks the gradient buckets
        loss = torch.nn.functional.cross_entropy(logits.flatten(0, 1).float(), targets.flatten())
        loss.backward()                                      # gradients are averaged by the backend
        optimizer.step()
        history.append(float(loss.detach()))

    prints = [None] * world
    dist.all_gather_object(prints, fingerprint(model))
    agree = len(set(prints)) == 1
    if rank == 0:
        verdict = "all replicas identical" if agree else f"REPLICAS DIFFER: {prints}"
        print(f"world {world} on {device.type}: loss {history[0]:.3f} -> {history[-1]:.3f}; {verdict}")
    dist.destroy_process_group()
    return 0 if agree else 1


if __name__ == "__main__":
    sys.exit(main())
