"""Process groups built straight from a c10d Store.

Every communicator the library owns (the Gloo group of all members, each island's native
group, a bridge's group of leaders) is a raw c10d backend object constructed from a
``PrefixStore``.  Only the members of a group construct it and nothing else in the job has
to take part, so no global ``dist.new_group`` ordering is needed and torch's private group
naming is never touched (the reference creates every group with ``dist.new_group`` on every
rank and patches ``distributed_c10d._process_group_name`` for subgroups:
src/gpubridge/topology.py:563-566, 645-692).

:class:`Comm` wraps such a backend with *global* rank arguments, which is what the
collective policies speak.
"""
from __future__ import annotations

import threading
from collections.abc import Sequence
from datetime import timedelta

import torch
import torch.distributed as dist

DEFAULT_TIMEOUT = timedelta(minutes=30)

_OPS = {"sum": dist.ReduceOp.SUM, "max": dist.ReduceOp.MAX, "min": dist.ReduceOp.MIN}


def reduce_op(name) -> dist.ReduceOp:
    if isinstance(name, str):
        return _OPS[name]
    return name


class Comm:
    """One communicator of ``ranks`` (global, ascending) as seen by member ``rank``."""

    def __init__(self, backend, ranks: Sequence[int], rank: int, kind: str, name: str = ""):
        self.backend = backend
        self.ranks = tuple(ranks)
        self.rank = rank
        self.kind = kind            # "gloo" | "nccl"
        self.name = name
        self.index = self.ranks.index(rank)
        self._lock = threading.Lock()

    # -- identity -------------------------------------------------------------------------
    @property
    def size(self) -> int:
        return len(self.ranks)

    @property
    def native(self) -> bool:
        """True for NCCL, which has the flat-tensor collectives built in."""
        return self.kind == "nccl"

    def local(self, global_rank: int) -> int:
        return self.ranks.index(global_rank)

    def __repr__(self) -> str:
        return f"Comm({self.kind}, ranks={list(self.ranks)}, rank={self.rank})"

    # -- collectives (blocking on the host for Gloo, stream-ordered for NCCL) -----------------
    def all_reduce(self, tensor: torch.Tensor, op="sum", async_op: bool = False):
        opts = dist.AllreduceOptions()
        opts.reduceOp = reduce_op(op)
        return self._finish(self.backend.allreduce([tensor], opts), async_op)

    def reduce(self, tensor: torch.Tensor, dst: int, op="sum", async_op: bool = False):
        opts = dist.ReduceOptions()
        opts.reduceOp = reduce_op(op)
        opts.rootRank = self.local(dst)
        return self._finish(self.backend.reduce([tensor], opts), async_op)

    def broadcast(self, tensor: torch.Tensor, src: int, async_op: bool = False):
        opts = dist.BroadcastOptions()
        opts.rootRank = self.local(src)
        opts.rootTensor = 0
        return self._finish(self.backend.broadcast([tensor], opts), async_op)

    def gather(self, tensor: torch.Tensor, rows: list[torch.Tensor] | None, dst: int):
        opts = dist.GatherOptions()
        opts.rootRank = self.local(dst)
        outputs = [rows] if rows is not None else []
        return self._finish(self.backend.gather(outputs, [tensor], opts), False)

    def scatter(self, tensor: torch.Tensor, slices: list[torch.Tensor] | None, src: int):
        opts = dist.ScatterOptions()
        opts.rootRank = self.local(src)
        inputs = [slices] if slices is not None else []
        return self._finish(self.backend.scatter([tensor], inputs, opts), False)

    def all_gather_into(self, output: torch.Tensor, tensor: torch.Tensor,
                        async_op: bool = False):
        """``output`` = every member's ``tensor`` back to back, in member order."""
        return self._finish(self.backend._allgather_base(output.view(-1), tensor.reshape(-1)),
                            async_op)

    def reduce_scatter_into(self, output: torch.Tensor, tensor: torch.Tensor, op="sum",
                            async_op: bool = False):
        """Member i keeps slice i of the reduction; ``tensor`` is left unmodified."""
        if self.native:
            opts = dist.ReduceScatterOptions()
            opts.reduceOp = reduce_op(op)
            return self._finish(self.backend._reduce_scatter_base(
                output.view(-1), tensor.reshape(-1), opts), async_op)
        # Gloo's reduce_scatter only sums; reduce a copy and slice it for MAX/MIN.
        work = tensor.reshape(-1).clone()
        self.all_reduce(work, op)
        output.view(-1).copy_(work.view(self.size, -1)[self.index])
        return None

    def barrier(self):
        return self._finish(self.backend.barrier(), False)

    def send(self, tensor: torch.Tensor, dst: int, tag: int = 0):
        return self.backend.send([tensor], self.local(dst), tag)

    def recv(self, tensor: torch.Tensor, src: int, tag: int = 0):
        return self.backend.recv([tensor], self.local(src), tag)

    def close(self) -> None:
        backend, self.backend = self.backend, None
        if backend is not None and self.kind == "nccl":
            try:
                backend.shutdown()
            except Exception:  # noqa: BLE001 - teardown never raises
                pass

    @staticmethod
    def _finish(work, async_op: bool):
        if async_op:
            return work
        work.wait()
        return None


def make_comm(store, name: str, ranks: Sequence[int], rank: int, kind: str,
              timeout: timedelta | None = None, device: torch.device | None = None
              ) -> Comm | None:
    """Construct the communicator ``name`` over ``ranks`` on its members; None elsewhere.

    Only members touch the store, under a prefix derived from ``name`` and the member list,
    so two groups can never meet on one key.  A single-member group gets a real backend too
    (Gloo and NCCL both accept size 1), which keeps every code path uniform.
    """
    ranks = tuple(ranks)
    if rank not in ranks:
        return None
    timeout = timeout or DEFAULT_TIMEOUT
    prefix = dist.PrefixStore(f"gb/{name}/{'_'.join(map(str, ranks))}", store)
    index = ranks.index(rank)
    if kind == "gloo":
        backend = dist.ProcessGroupGloo(prefix, index, len(ranks), timeout)
    elif kind == "nccl":
        options = dist.ProcessGroupNCCL.Options()
        options._timeout = timeout
        # The NCCL communicator itself connects at the group's first collective.
        backend = dist.ProcessGroupNCCL(prefix, index, len(ranks), options)
    else:
        raise ValueError(f"unknown communicator kind {kind!r}")
    return Comm(backend, ranks, rank, kind, name)
