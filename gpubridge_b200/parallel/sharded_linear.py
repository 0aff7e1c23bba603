"""A Linear layer whose weight lives sharded by output rows over the data-parallel group - the
way FSDP2 shards it - with the all-gather fused into the forward GEMM.

Stock FSDP2 runs ``all_gather_into_tensor(weight shards)`` and then ``F.linear`` (reference:
src/gpubridge/torch_backend.py:271-285 carries the all-gather).  Here, on GPUs that share a
fabric, forward is one kernel (``csrc/gb_gemm*.cu``): communication CTAs bring the peers'
shards over NVLink while tcgen05 GEMM CTAs already multiply the local shard, and take each
remote shard as soon as its flag is up.  Backward reuses the gathered weight that forward
left in local memory for ``dX = dY @ W`` and reduce-scatters ``dW = dY^T @ X`` so that every
rank ends with the averaged gradient of its own rows.  Without a fabric (CPU simulation,
several hosts) the same module all-gathers through the collectives and calls ``F.linear``.

    layer = ShardedLinear(4096, 14336)          # every rank holds 14336 / world rows
    y = layer(x)                                # x: [tokens, 4096], y: [tokens, 14336]
"""
from __future__ import annotations

import math

import torch
from torch import nn
from torch.distributed import ReduceOp

from gpubridge_b200 import collectives
from gpubridge_b200.topology import Topology, get_topology, is_initialized


class _FusedForward(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, shard, layer):
        x2 = x.reshape(-1, x.shape[-1])
        y = layer._gemm(x2.contiguous(), shard.contiguous())
        ctx.layer = layer
        ctx.save_for_backward(x2)
        return y.view(*x.shape[:-1], y.shape[-1])

    @staticmethod
    def backward(ctx, dy):
        layer = ctx.layer
        (x2,) = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        weight = layer._gathered()                       # left in local memory by forward
        dx = (dy2 @ weight).view(*dy.shape[:-1], weight.shape[1]) if ctx.needs_input_grad[0] else None
        dshard = None
        if ctx.needs_input_grad[1]:
            dw = (dy2.t() @ x2).contiguous()             # [N, K], this rank's contribution
            dshard = layer._scatter_gradient(dw)
        return dx, dshard, None


class ShardedLinear(nn.Module):
    """``y = x @ W^T`` with ``W`` [out_features, in_features] sharded by rows; no bias.  The
    parameter is this rank's shard; its gradient is the average over ranks of the rows it
    owns (what FSDP2's reduce-scatter leaves)."""

    def __init__(self, in_features: int, out_features: int, *, topology: Topology | None = None,
                 device=None, dtype=torch.bfloat16, seed: int = 0) -> None:
        super().__init__()
        if topology is None and is_initialized():
            topology = get_topology()
        self.topology = topology
        self.world = topology.world_size if topology is not None else 1
        self.rank = topology.rank if topology is not None else 0
        if out_features % self.world:
            raise ValueError(f"out_features ({out_features}) must divide over {self.world} ranks")
        self.in_features, self.out_features = in_features, out_features
        device = device or (topology.device if topology is not None else "cpu")
        rows = out_features // self.world
        # every rank draws the whole weight from one seed and keeps its rows: the same model
        # for any world size
        g = torch.Generator().manual_seed(seed)
        full = torch.empty(out_features, in_features).uniform_(-1, 1, generator=g) / math.sqrt(in_features)
        self.weight = nn.Parameter(full[self.rank * rows:(self.rank + 1) * rows].to(device=device, dtype=dtype))
        self._op = None
        self._full = None

    # -- the three pieces ---------------------------------------------------------------------
    def _fused(self) -> bool:
        fabric = self.topology.fabric if self.topology is not None else None
        return (fabric is not None and self.weight.is_cuda and self.weight.dtype == torch.bfloat16
                and self.in_features % 8 == 0)

    def _gemm(self, x2: torch.Tensor, shard: torch.Tensor) -> torch.Tensor:
        if self._fused():
            if self._op is None:
                from gpubridge_b200.ops.gemm import AllGatherLinear
                self._op = AllGatherLinear(self.topology.fabric, self.out_features, self.in_features)
            return self._op(x2.to(torch.bfloat16), shard)
        if self.world == 1:
            self._full = shard
        else:
            self._full = torch.empty((self.out_features, self.in_features), dtype=shard.dtype,
                                     device=shard.device)
            collectives.all_gather_into_tensor(self._full, shard, _topology=self.topology)
        return torch.nn.functional.linear(x2, self._full)

    def _gathered(self) -> torch.Tensor:
        return self._op.gathered if self._op is not None else self._full

    def _scatter_gradient(self, dw: torch.Tensor) -> torch.Tensor:
        if self.world == 1:
            return dw
        out = torch.empty_like(self.weight)
        collectives.reduce_scatter_tensor(out, dw, ReduceOp.AVG, _topology=self.topology)
        return out

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return _FusedForward.apply(x, self.weight, self)
