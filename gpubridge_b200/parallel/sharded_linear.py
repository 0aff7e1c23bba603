"""A Linear layer whose weight lives sharded by output rows over the data-parallel group - the
way FSDP2 shards it - with the all-gather fused into the forward GEMM.

Stock FSDP2 runs ``all_gather_into_tensor(weight shards)`` and then ``F.linear`` (reference:
src/gpubridge/torch_backend.py:271-285 carries the all-gather).  Here, on GPUs that share a
fabric, forward is one kernel (``csrc/gb_gemm*.cu``): communication CTAs bring the peers'
shards over NVLink while tcgen05 GEMM CTAs already multiply the local shard, and take each
remote shard as soon as its flag is up.  Backward needs the whole weight once more for
``dX = dY @ W`` and reduce-scatters ``dW = dY^T @ X`` so that every rank ends with the
averaged gradient of its own rows.  Without a fabric (CPU simulation, several hosts) the same
module all-gathers through the collectives and calls ``F.linear``.

Memory is what makes sharding worth it, so the gathered weight is not the layer's: layers of
one shape (and dtype) on one topology share one *slot*, the way FSDP2 reshards after forward.
Forward gathers into the slot and marks it as this call's; backward uses it as it is when
nothing else has gathered into it since (the last layer of a stack, a layer on its own) and
gathers again otherwise (one fused copy kernel over NVLink).  A stack of L equal layers holds
one whole weight, not L.  ``reshard_after_forward=False`` gives a layer a slot of its own:
no second gather, a whole weight resident per layer.

    layer = ShardedLinear(4096, 14336)          # every rank holds 14336 / world rows
    y = layer(x)                                # x: [tokens, 4096], y: [tokens, 14336]
"""
from __future__ import annotations

import math
import os
import weakref

import torch
from torch import nn
from torch.distributed import ReduceOp

from gpubridge_b200 import collectives
from gpubridge_b200.topology import Topology, get_topology, is_initialized


class GatherSlot:
    """One whole weight's worth of memory and the record of whose gather it holds."""

    def __init__(self, topology) -> None:
        self.topology = weakref.ref(topology) if topology is not None else None
        self.buffer: torch.Tensor | None = None
        self.op = None                      # the fused all-gather GEMM site bound to ``buffer``
        self.scatter = None                 # the fused GEMM + reduce-scatter of the weight gradient
        self.holder: object | None = None   # token of the forward call whose weight is in it
        self.gathers = 0                    # gathers into this slot, forward and backward (tests)


_slots: dict[tuple, GatherSlot] = {}


def _slot_for(topology, key: tuple) -> GatherSlot:
    """The shared slot of ``key`` on ``topology``.  The table is keyed by the topology's id;
    the weak reference tells a live topology from a new one that got a dead one's id."""
    full_key = (id(topology), *key)
    slot = _slots.get(full_key)
    if slot is None or (slot.topology is not None and slot.topology() is not topology):
        slot = _slots[full_key] = GatherSlot(topology)
    return slot


def release_slots(topology=None) -> None:
    """Drop the shared slots of ``topology`` (all of them by default): frees their memory."""
    for key in [k for k in _slots if topology is None or k[0] == id(topology)]:
        del _slots[key]


class _FusedForward(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, shard, layer):
        x2 = x.reshape(-1, x.shape[-1])
        ctx.token = object()
        y = layer._gemm(x2.contiguous(), shard.contiguous(), ctx.token)
        ctx.layer = layer
        ctx.save_for_backward(x2, shard)
        return y.view(*x.shape[:-1], y.shape[-1])

    @staticmethod
    def backward(ctx, dy):
        layer = ctx.layer
        x2, shard = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        weight = layer._gathered(shard, ctx.token)       # still in the slot, or gathered again
        dx = (dy2 @ weight).view(*dy.shape[:-1], weight.shape[1]) if ctx.needs_input_grad[0] else None
        dshard = None
        if ctx.needs_input_grad[1]:
            dshard = layer._weight_gradient(dy2, x2)
        return dx, dshard, None


class ShardedLinear(nn.Module):
    """``y = x @ W^T`` with ``W`` [out_features, in_features] sharded by rows; no bias.  The
    parameter is this rank's shard; its gradient is the average over ranks of the rows it
    owns (what FSDP2's reduce-scatter leaves)."""

    def __init__(self, in_features: int, out_features: int, *, topology: Topology | None = None,
                 device=None, dtype=torch.bfloat16, seed: int = 0,
                 reshard_after_forward: bool = True) -> None:
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
        self.reshard_after_forward = reshard_after_forward
        self._own_slot = None if reshard_after_forward else GatherSlot(topology)
        self.grad_chunks = int(os.environ.get("GPUBRIDGE_SHARDED_GRAD_CHUNKS", "1"))
        self.fused_gradient = os.environ.get("GPUBRIDGE_GEMM_RS", "0") == "1"

    @classmethod
    def from_linear(cls, linear: nn.Linear, topology: Topology | None = None,
                    reshard_after_forward: bool = True) -> "ShardedLinear":
        """A sharded layer holding this rank's rows of ``linear.weight`` (every rank passes the
        same whole weight, e.g. a model built from one seed).  ``linear`` must have no bias."""
        if linear.bias is not None:
            raise ValueError("ShardedLinear has no bias")
        layer = cls.__new__(cls)
        nn.Module.__init__(layer)
        if topology is None and is_initialized():
            topology = get_topology()
        layer.topology = topology
        layer.world = topology.world_size if topology is not None else 1
        layer.rank = topology.rank if topology is not None else 0
        layer.out_features, layer.in_features = linear.weight.shape
        if layer.out_features % layer.world:
            raise ValueError(f"out_features ({layer.out_features}) must divide over {layer.world} ranks")
        rows = layer.out_features // layer.world
        layer.weight = nn.Parameter(linear.weight.detach()[layer.rank * rows:(layer.rank + 1) * rows].clone())
        layer.reshard_after_forward = reshard_after_forward
        layer._own_slot = None if reshard_after_forward else GatherSlot(topology)
        layer.grad_chunks = int(os.environ.get("GPUBRIDGE_SHARDED_GRAD_CHUNKS", "1"))
        layer.fused_gradient = os.environ.get("GPUBRIDGE_GEMM_RS", "0") == "1"
        return layer

    # -- the three pieces ---------------------------------------------------------------------
    #: Largest weight (elements) for which the one-kernel all-gather + GEMM is the default.
    #: Measured on four B200s: at 5632 x 2048 and 8192 rows of input the fused kernel takes 300 us
    #: against 244-279 us for an all-gather followed by cuBLAS (its GEMM runs at 0.6 of cuBLAS);
    #: at 2048 x 1024 on two it takes 57 us against 76 us (one launch and one barrier less).
    FUSED_MAX_WEIGHT = 4 << 20

    def _fused(self) -> bool:
        """Whether forward runs the fused all-gather + GEMM kernel.  ``GPUBRIDGE_GEMM_FUSED``:
        ``1`` always (where it can), ``0`` never, unset: for weights up to ``FUSED_MAX_WEIGHT``
        elements, where a launch and a barrier saved weigh more than the slower GEMM."""
        fabric = self.topology.fabric if self.topology is not None else None
        able = (fabric is not None and self.weight.is_cuda and self.weight.dtype == torch.bfloat16
                and self.in_features % 8 == 0)
        choice = os.environ.get("GPUBRIDGE_GEMM_FUSED", "")
        if not able or choice == "0":
            return False
        return choice == "1" or self.out_features * self.in_features <= self.FUSED_MAX_WEIGHT

    def _slot(self) -> GatherSlot:
        if self._own_slot is not None:
            return self._own_slot
        return _slot_for(self.topology, (self.out_features, self.in_features, self.weight.dtype,
                                         str(self.weight.device), self._fused()))

    def _buffer(self, slot: GatherSlot) -> torch.Tensor:
        if slot.buffer is None:
            slot.buffer = torch.empty((self.out_features, self.in_features), dtype=self.weight.dtype,
                                      device=self.weight.device)
        return slot.buffer

    def _gemm(self, x2: torch.Tensor, shard: torch.Tensor, token: object) -> torch.Tensor:
        if self.world == 1 and not self._fused():
            return torch.nn.functional.linear(x2, shard)
        slot = self._slot()
        full = self._buffer(slot)
        slot.holder, slot.gathers = token, slot.gathers + 1
        if self._fused():
            if slot.op is None:
                from gpubridge_b200.ops.gemm import AllGatherLinear
                slot.op = AllGatherLinear(self.topology.fabric, self.out_features, self.in_features,
                                          gathered=full)
            return slot.op(x2.to(torch.bfloat16), shard)
        collectives.all_gather_into_tensor(full, shard, _topology=self.topology)
        return torch.nn.functional.linear(x2, full)

    def _gathered(self, shard: torch.Tensor, token: object) -> torch.Tensor:
        """The whole weight for backward: what forward left in the slot if it is still this
        call's, else gathered again."""
        if self.world == 1 and not self._fused():
            return shard
        slot = self._slot()
        full = self._buffer(slot)
        if slot.holder is not token:
            collectives.all_gather_into_tensor(full, shard.contiguous(), _topology=self.topology)
            slot.holder, slot.gathers = token, slot.gathers + 1
        return full

    def _weight_gradient(self, dy2: torch.Tensor, x2: torch.Tensor) -> torch.Tensor:
        """This rank's rows of the averaged ``dW = dY^T @ X``.

        ``GPUBRIDGE_GEMM_RS=1``: on the fused path, one kernel (``csrc/gb_gemm_rs.cu``) whose
        epilogue sends every row of the product to its owner.  Otherwise
        ``GPUBRIDGE_SHARDED_GRAD_CHUNKS`` (default 1) cuts every owner's rows into that many
        pieces: piece s of all owners is one batched GEMM into a contiguous [world, rows / S, K]
        buffer and one asynchronous reduce-scatter, so the exchange of piece s runs on the
        communication stream (on few CTAs) while the GEMM of piece s + 1 runs - the overlap a
        single GEMM -> reduce-scatter kernel would give tile by tile, from two kernels."""
        if self.world == 1:
            return (dy2.t() @ x2).contiguous()
        if self.fused_gradient and self._fused() and dy2.dtype == torch.bfloat16 == x2.dtype:
            # one kernel: the GEMM's epilogue sends every row to its owner, a reducing tail follows
            slot = self._slot()
            if slot.scatter is None:
                from gpubridge_b200.ops.gemm import GemmReduceScatter
                slot.scatter = GemmReduceScatter(self.topology.fabric)
            if slot.scatter.fits(self.out_features, self.in_features, dy2.shape[0]):
                return slot.scatter(dy2.t().contiguous(), x2.t().contiguous(), divide=self.world,
                                    out_dtype=self.weight.dtype)
        out = torch.empty_like(self.weight)
        rows = self.out_features // self.world
        pieces = max(1, min(self.grad_chunks, rows))
        if pieces == 1 or rows % pieces:
            dw = (dy2.t() @ x2).contiguous()             # [N, K], this rank's contribution
            collectives.reduce_scatter_tensor(out, dw, ReduceOp.AVG, _topology=self.topology)
            return out
        per = rows // pieces
        dyt = dy2.t().reshape(self.world, rows, dy2.shape[0])            # [owner, row, token]
        works = []
        for s in range(pieces):
            part = torch.matmul(dyt[:, s * per:(s + 1) * per, :], x2)    # [owner, per, K]
            works.append(collectives.reduce_scatter_tensor(
                out[s * per:(s + 1) * per], part.contiguous(), ReduceOp.AVG, async_op=True,
                _topology=self.topology))
        for work in works:
            work.wait()
        return out

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return _FusedForward.apply(x, self.weight, self)
