"""Shard a model's Linear layers over the data-parallel group, FSDP-style, on the fused
all-gather GEMM - and keep everything else replicated and in sync.

    model = llama.build("llama-1b", device=device)
    plan = shard_linears(model.blocks, topology)        # every bias-free nn.Linear -> ShardedLinear
    sync = ReplicatedSync(model, topology)              # the parameters that stayed whole
    ...
    loss.backward()
    sync.average_gradients()                            # one flat all-reduce (AVG) for the rest
    optimizer.step()

What FSDP2 does with hooks around every module - all-gather the parameters, run the module,
free them, reduce-scatter the gradients (reference: the collectives of
src/gpubridge/torch_backend.py:271-310 carry it) - a :class:`ShardedLinear` does inside its
own forward and backward: the all-gather is fused into the tcgen05 GEMM, the reduce-scatter
averages its weight gradient, and layers of one shape share one gathered-weight slot.  The
parameters that are not Linear weights (embeddings, norms, an output layer whose rows do not
divide) stay replicated; their gradients are averaged with one all-reduce of a flat buffer.

Memory per rank: Linear weights / world, plus one whole weight per distinct layer shape, plus
the replicated rest - against the whole model for plain data parallel.
"""
from __future__ import annotations

import torch
from torch import nn
from torch.distributed import ReduceOp

from gpubridge_b200 import collectives
from gpubridge_b200.parallel.sharded_linear import ShardedLinear
from gpubridge_b200.topology import Topology


def shard_linears(root: nn.Module, topology: Topology | None, *, min_features: int = 0,
                  reshard_after_forward: bool = True) -> dict[str, tuple[int, int]]:
    """Replace, in place, every bias-free ``nn.Linear`` under ``root`` whose output rows divide
    over the group (and are at least ``min_features``) with a :class:`ShardedLinear` holding this
    rank's rows.  Every rank must call it on an identical model.  Returns ``{name: (out, in)}``
    of what was sharded."""
    world = topology.world_size if topology is not None else 1
    done: dict[str, tuple[int, int]] = {}
    for name, module in list(root.named_modules()):
        for child_name, child in list(module.named_children()):
            if (isinstance(child, nn.Linear) and child.bias is None and child.out_features % world == 0
                    and child.out_features >= min_features):
                setattr(module, child_name, ShardedLinear.from_linear(
                    child, topology, reshard_after_forward=reshard_after_forward))
                done[f"{name}.{child_name}".lstrip(".")] = (child.out_features, child.in_features)
    return done


class ReplicatedSync:
    """Averages, over the group, the gradients of the parameters that stayed whole."""

    def __init__(self, model: nn.Module, topology: Topology | None) -> None:
        sharded = {id(m.weight) for m in model.modules() if isinstance(m, ShardedLinear)}
        self.topology = topology
        self.params = [p for p in model.parameters() if p.requires_grad and id(p) not in sharded]
        self.numel = sum(p.numel() for p in self.params)
        self._flat: torch.Tensor | None = None

    def average_gradients(self) -> None:
        if self.topology is None or self.topology.world_size == 1 or not self.params:
            return
        first = self.params[0]
        if self._flat is None:
            self._flat = torch.zeros(self.numel, dtype=torch.float32, device=first.device)
        flat, offset = self._flat, 0
        for p in self.params:                    # pack (a parameter without a gradient counts as zero)
            view = flat[offset:offset + p.numel()]
            if p.grad is None:
                view.zero_()
            else:
                view.copy_(p.grad.reshape(-1))
            offset += p.numel()
        collectives.all_reduce(flat, ReduceOp.AVG, _topology=self.topology)
        offset = 0
        for p in self.params:
            if p.grad is not None:
                p.grad.copy_(flat[offset:offset + p.numel()].view_as(p.grad))
            offset += p.numel()

    def memory(self, model: nn.Module) -> dict[str, int]:
        """Bytes of parameters this rank holds: sharded rows, replicated rest."""
        sharded = sum(m.weight.numel() * m.weight.element_size() for m in model.modules()
                      if isinstance(m, ShardedLinear))
        rest = sum(p.numel() * p.element_size() for p in self.params)
        return {"sharded_bytes": sharded, "replicated_bytes": rest}
