"""Data-parallel training step built on the fabric: flat buffers, bucketed gradient
all-reduce overlapped with backward, fused AdamW, optionally replayed from a CUDA graph.

This is the B200-first counterpart of "DistributedDataParallel + ``ddp_comm_hook`` +
``torch.optim.AdamW``" (reference: src/gpubridge/ddp.py:41-52 and the training loop of
scripts/gpu/train_bench.py:300-330).  The hook path still exists
(:func:`gpubridge_b200.ddp_comm_hook`); this trainer is what a user calls when the whole
step should be ours:

* every parameter is a view into one flat float32 buffer, every gradient a view into
  another, so the optimizer is one launch (``csrc/gb_optim.cu``) that also clears the
  gradients;
* gradients are cut into buckets in reverse registration order (the order backward
  produces them); when the last gradient of a bucket has been accumulated, the bucket's
  all-reduce (AVG fused, hierarchical, optionally compressed on the cross-island leg) is
  launched on the fabric's communication stream while backward continues;
* none of this needs the host between launches, and the collective kernels keep their
  sequence numbers on the device, so the whole step - forward, backward, collectives,
  optimizer - can be captured once and replayed as one CUDA graph on every rank.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from gpubridge_b200.ops.optim import FlatAdamW
from gpubridge_b200.topology import Topology, get_topology, is_initialized

MIB = 1 << 20


class DataParallelTrainer:
    """One training step per :meth:`step` call.

    Args:
        model: the module to train; its parameters are moved into the flat buffer.
        loss_fn: ``loss_fn(model, *batch) -> scalar loss``.
        topology: the group to average gradients over (default: the initialised world;
            None and not initialised: a single process).
        bucket_mb: gradient bucket size (DDP's default is 25 MB).
        autocast: dtype of ``torch.autocast`` around forward, or None.
        graph: capture the step in a CUDA graph after ``graph_warmup`` eager steps.
        overlap_blocks: CTAs of a bucket all-reduce that runs beside backward
            (``GPUBRIDGE_OVERLAP_BLOCKS``; default 16 when the gradients live in switch memory,
            else 32); the last bucket uses the full grid.
        unit_grad: tell a model that has a ``unit_grad`` switch that backward starts at its
            loss with gradient 1 (its fused loss then skips the multiply); pass False when
            ``loss_fn`` scales the model's loss.
        exchange: False trains this rank alone even inside an initialised job (the
            compute-only phase of a benchmark).
        optimizer_in_backward: update a bucket's parameters as soon as its averaged gradients
            are there, on a side stream beside the rest of backward (the layers a bucket
            belongs to have finished their backward by then, so nothing reads those
            parameters again before the next forward); only the last bucket's update is left
            for after backward.  The arithmetic and its result are those of one optimizer
            call after backward.  ``GPUBRIDGE_OPTIMIZER_IN_BACKWARD``: ``1``, ``0``, or unset =
            on a team of two or more only (alone it costs more than it hides).
    """

    def __init__(self, model: nn.Module, loss_fn, *, topology: Topology | None = None,
                 lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8,
                 weight_decay: float = 1e-2, bucket_mb: float = 25.0,
                 autocast: torch.dtype | None = torch.bfloat16, graph: bool = False,
                 graph_warmup: int = 3, overlap_blocks: int | None = None,
                 unit_grad: bool = True, exchange: bool = True,
                 optimizer_in_backward: bool | None = None) -> None:
        self.model, self.loss_fn = model, loss_fn
        import os
        self.overlap_blocks = overlap_blocks or int(os.environ.get("GPUBRIDGE_OVERLAP_BLOCKS", "0"))
        self._in_backward_wanted = optimizer_in_backward
        # grid of an update that runs beside backward (the last bucket's takes what it wants)
        self.update_blocks = int(os.environ.get("GPUBRIDGE_UPDATE_BLOCKS", "0"))
        if hasattr(model, "unit_grad"):
            model.unit_grad = unit_grad     # backward always starts at the loss here
        if not exchange:
            topology = None
        elif topology is None and is_initialized():
            topology = get_topology()
        self.topology = topology
        self.world = topology.world_size if topology is not None else 1
        self.fabric = topology.fabric if topology is not None else None
        self.autocast = autocast
        params = [p for p in model.parameters() if p.requires_grad]
        self.device = params[0].device
        sizes = [-(-p.numel() // 64) * 64 for p in params]          # 256-byte aligned views
        total = sum(sizes)
        self.flat_param = torch.zeros(total, dtype=torch.float32, device=self.device)
        # The gradients live in the team's switch memory when it has some: bucket all-reduces
        # then run in place inside the NVSwitch (no staging copies, a handful of SMs), which is
        # what lets them hide under backward.  Collective: every rank builds its trainer.
        in_switch = None
        if self.fabric is not None and self.world > 1 and hasattr(self.fabric, "switch_empty"):
            in_switch = self.fabric.switch_empty(total, torch.float32)
        self.grads_in_switch = in_switch is not None
        if not self.overlap_blocks:
            # measured: in place in the switch 8-16 CTAs keep up with the buckets and cost
            # backward the least (four B200s: 14.67 / 14.69 ms a step with 8 / 16 against 14.80
            # with 32; two: 14.88 / 14.67 with 8 / 16); the peer-memory kernels need their 32
            self.overlap_blocks = 16 if self.grads_in_switch else 32
        # Alone, an update beside backward costs more than it hides (13.7 ms a step after
        # backward, 14.3-14.9 inside it: every kernel that shares the GPU delays cuBLAS's
        # persistent GEMMs); on a team the updates follow the bucket all-reduces, which are
        # there anyway, and the step gets about 0.1 ms shorter.
        wanted = self._in_backward_wanted
        if wanted is None:
            wanted = os.environ.get("GPUBRIDGE_OPTIMIZER_IN_BACKWARD", "auto")
            wanted = self.world > 1 if wanted == "auto" else wanted == "1"
        self.optimizer_in_backward = bool(wanted)
        self.flat_grad = in_switch if in_switch is not None else \
            torch.zeros(total, dtype=torch.float32, device=self.device)
        # reverse registration order: the order backward fills the gradients in
        offset, self._spans = 0, []
        for p, size in zip(reversed(params), reversed(sizes)):
            view = self.flat_param[offset:offset + p.numel()].view_as(p)
            view.copy_(p.detach())
            p.data = view
            p.grad = self.flat_grad[offset:offset + p.numel()].view_as(p)
            self._spans.append((p, offset, offset + size))
            offset += size
        self.optimizer = FlatAdamW(self.flat_param, self.flat_grad, lr, betas, eps, weight_decay)
        self._buckets = self._make_buckets(int(bucket_mb * MIB))
        self._pending = [0] * len(self._buckets)
        self._sent = 0
        self._syncing = True
        self._comm_events: list[torch.cuda.Event] = []
        # the bucket updates of an optimizer that runs inside backward get a stream of their own
        self._opt_stream = (torch.cuda.Stream(self.device)
                            if self.optimizer_in_backward and self.device.type == "cuda" else None)
        if self.world > 1 or self.optimizer_in_backward:
            for index, (lo, hi, members) in enumerate(self._buckets):
                for p in members:
                    p.register_post_accumulate_grad_hook(self._make_hook(index))
        self._use_graph, self._graph_warmup = graph and self.device.type == "cuda", graph_warmup
        self._graph: torch.cuda.CUDAGraph | None = None
        self._static_batch = None
        self._static_loss = None
        self._steps = 0
        self.launches = 0

    # -- buckets -------------------------------------------------------------------------------
    def _make_buckets(self, cap_bytes: int):
        buckets, lo, members = [], 0, []
        for p, start, end in self._spans:
            members.append(p)
            if (end - lo) * 4 >= cap_bytes:
                buckets.append((lo, end, members))
                lo, members = end, []
        if members:
            buckets.append((lo, self._spans[-1][2], members))
        return buckets

    def _make_hook(self, index: int):
        def hook(param) -> None:
            if not self._syncing:           # an earlier micro-batch: gradients only accumulate
                return
            self._pending[index] -= 1
            if self._pending[index] == 0:
                self._reduce_ready()
        return hook

    def _reduce_ready(self) -> None:
        """Launch, in bucket order, every bucket whose gradients are all in."""
        while self._sent < len(self._buckets) and self._pending[self._sent] == 0:
            lo, hi, _ = self._buckets[self._sent]
            tail = self._sent == len(self._buckets) - 1
            if self.world > 1:
                self._all_reduce(self.flat_grad[lo:hi], tail=tail)
            if self.optimizer_in_backward:
                self._update(lo, hi, tail)
            self._sent += 1

    def _update(self, lo: int, hi: int, last: bool) -> None:
        """The optimizer on one bucket, ordered after the bucket's all-reduce (or, alone, after
        the backward so far) and beside whatever backward still has to do."""
        side = self._opt_stream
        if side is None:
            self.optimizer.step_span(lo, hi, last=last, zero_grad=True)
            return
        after = self.fabric.comm_stream if self.world > 1 and self.fabric is not None \
            else torch.cuda.current_stream(self.device)
        side.wait_stream(after)
        with torch.cuda.stream(side):
            self.optimizer.step_span(lo, hi, last=last, zero_grad=True,
                                     max_blocks=0 if last else self.update_blocks)

    def _all_reduce(self, grads: torch.Tensor, tail: bool = False) -> None:
        topology, fabric = self.topology, self.fabric
        if fabric is not None:
            # stream-ordered: fork onto the communication stream, join before the optimizer.
            # A bucket that runs beside backward takes few SMs (a CTA of the collective owns
            # its SM, so a full grid would serialise with the GEMMs instead of overlapping);
            # the last bucket has nothing left to overlap with and takes the full grid.
            comm = fabric.comm_stream
            comm.wait_stream(torch.cuda.current_stream(self.device))
            with fabric.grid_cap(None if tail else self.overlap_blocks), torch.cuda.stream(comm):
                topology.policy.select_policy(grads.nbytes).all_reduce(
                    grads, topology, divide=self.world)
        else:
            from gpubridge_b200.collectives import all_reduce
            from torch.distributed import ReduceOp
            all_reduce(grads, ReduceOp.AVG, _topology=topology)

    # -- the step --------------------------------------------------------------------------------
    def _own_kernels(self) -> int:
        """Launches of this library's kernels so far (every op module keeps a counter)."""
        from gpubridge_b200.ops import layernorm, optim, xent
        total = layernorm.launches + optim.launches + xent.launches
        if self.fabric is not None:
            total += self.fabric.launches
        return total

    def _step_body(self, batch, earlier=()) -> torch.Tensor:
        own_before = self._own_kernels()
        self._pending = [len(members) for _, _, members in self._buckets]
        self._sent = 0
        total = None
        for micro in (*earlier, batch):
            self._syncing = micro is batch
            if self.autocast is not None and self.device.type == "cuda":
                with torch.autocast("cuda", dtype=self.autocast):
                    loss = self.loss_fn(self.model, *micro)
            else:
                loss = self.loss_fn(self.model, *micro)
            loss.backward()
            total = loss.detach() if total is None else total + loss.detach()
        loss = total
        if self.world > 1 or self.optimizer_in_backward:
            # parameters that received no gradient still belong to their bucket
            self._pending = [0] * len(self._buckets)
            self._reduce_ready()
            if self.world > 1 and self.fabric is not None:
                torch.cuda.current_stream(self.device).wait_stream(self.fabric.comm_stream)
        if not self.optimizer_in_backward:
            self.optimizer.step(zero_grad=True)
        elif self._opt_stream is not None:
            torch.cuda.current_stream(self.device).wait_stream(self._opt_stream)
        self.launches += self._own_kernels() - own_before
        return loss

    def step_accumulated(self, micro_batches) -> torch.Tensor:
        """One optimizer step over several micro-batches: forward and backward on each in
        turn, gradients summed in the flat buffer, buckets averaged once, during the last
        backward (what ``DistributedDataParallel.no_sync()`` does for the reference's
        ``--accumulate``, scripts/gpu/train_bench.py:57-68).  Runs eagerly.  Returns the sum
        of the micro-batch losses; weight them inside ``loss_fn`` so the sum is the loss
        wanted."""
        self._steps += 1
        moved = [[b.to(self.device, non_blocking=True) for b in micro] for micro in micro_batches]
        return self._step_body(moved[-1], earlier=moved[:-1])

    def step(self, *batch: torch.Tensor) -> torch.Tensor:
        """Forward, backward with overlapped gradient averaging, optimizer.  Returns the
        loss of this rank's batch as a device tensor (no host synchronisation)."""
        self._steps += 1
        if not self._use_graph or (self._graph is None and self._steps <= self._graph_warmup):
            return self._step_body([b.to(self.device, non_blocking=True) for b in batch])
        if self._graph is None:
            self._capture([b.to(self.device) for b in batch])
        for static, new in zip(self._static_batch, batch):
            static.copy_(new, non_blocking=True)
        before = self.launches
        self._graph.replay()
        self.launches = before + self._launches_per_step
        return self._static_loss

    def _capture(self, batch) -> None:
        self._static_batch = [b.clone() for b in batch]
        torch.cuda.synchronize(self.device)
        self._graph = torch.cuda.CUDAGraph()
        before = self.launches
        with torch.cuda.graph(self._graph):
            self._static_loss = self._step_body(self._static_batch)
        self._launches_per_step = self.launches - before
        self.launches = before

    def check(self) -> None:
        """Raise if a device-side wait of a collective ran out."""
        if self.fabric is not None:
            self.fabric.check()
