"""Collective policies: how a group-wide collective is put together.

The names, the contract and the semantics are the reference's
(src/gpubridge/policies.py:142-1064):

``native-only``                        one native collective on the only island
``reduce-bridge-broadcast``            island reduce -> leaders over the bridge -> island broadcast
``pipelined-reduce-bridge-broadcast``  the same, the bridge step cut into chunks
``sharded-bridge``                     k ranks per island share the bridge step, one stripe each
``flat-gloo``                          every rank through host memory on one Gloo group (the oracle)
``auto-tuned``                         one of the above by message size, from a thresholds file

``auto`` picks ``native-only`` for one island and ``reduce-bridge-broadcast`` otherwise.

Each bridged policy has two executions.  **Fused** (a GPU group on one NVSwitch box, i.e.
``topology.fabric`` is set): the whole collective is one launch of a hand-written sm_100a
kernel that reads and writes the peers' symmetric buffers over NVLink; the island reduce,
the leaders' exchange (compressed if asked), the island broadcast, AVG and the output cast
happen inside it.  "Pipelined" then means in-kernel chunking and "sharded" multi-leader
striping.  **Composed** (CPU simulation, several hosts, or ``GPUBRIDGE_FABRIC=off``): the
collective is assembled from island collectives and bridge-transport calls through host
memory, which is what the reference always does.  Both give every rank identical bits, and
exact results on integer-valued data.
"""
from __future__ import annotations

import abc
import dataclasses
import json
import os
from typing import TYPE_CHECKING, Any, ClassVar

import torch

from gpubridge_b200 import compression as _compression
from gpubridge_b200 import staging as _staging
from gpubridge_b200.config import THRESHOLDS_ENV, chunk_bytes_setting
from gpubridge_b200.observe import phase

if TYPE_CHECKING:
    from gpubridge_b200.topology import Layout, Topology
    from gpubridge_b200.transport import BridgeTransport

AUTO = "auto"
_ALL_OPS = frozenset({"sum", "max", "min"})


def _stage_to_host(tensor: torch.Tensor) -> torch.Tensor:
    """A host copy of ``tensor`` (itself on CPU).  Tests swap this for ``clone`` so the CPU
    run takes the copy-out-and-back path of a GPU."""
    return tensor.cpu()


def _host_like(tensor: torch.Tensor) -> torch.Tensor:
    if tensor.device.type == "cpu":
        return _stage_to_host(tensor)
    return torch.empty(tensor.shape, dtype=tensor.dtype)


class CollectivePolicy(abc.ABC):
    """How collectives travel.  One instance per rank and topology; every rank of a group
    runs the same class with the same settings, which is what keeps a policy from hanging."""

    name: ClassVar[str]
    reduce_ops: ClassVar[frozenset[str]] = frozenset({"sum"})

    @classmethod
    @abc.abstractmethod
    def applies_to(cls, layout: "Layout") -> bool: ...

    @abc.abstractmethod
    def all_reduce(self, tensor: torch.Tensor, topology: "Topology", op: str = "sum") -> None:
        """Reduce an already-validated tensor over every member, in place."""

    @abc.abstractmethod
    def broadcast(self, tensor: torch.Tensor, src: int, topology: "Topology") -> None:
        """Copy from global rank ``src`` to every member, in place."""

    def all_gather_into_tensor(self, output, input, topology) -> None:  # noqa: A002
        raise NotImplementedError(
            f"collective policy {self.name!r} doesn't implement all_gather_into_tensor")

    def reduce_scatter_tensor(self, output, input, topology) -> None:  # noqa: A002
        raise NotImplementedError(
            f"collective policy {self.name!r} doesn't implement reduce_scatter_tensor")

    def supported_reduce_ops(self, topology: "Topology") -> frozenset[str]:
        return self.reduce_ops

    @classmethod
    def settings(cls) -> dict[str, Any]:
        """Environment settings every rank must share (plain JSON values)."""
        return {}

    def setup(self, topology: "Topology") -> None:  # noqa: B027
        """Called once after every communicator exists."""

    def close(self) -> None:  # noqa: B027
        """Release what :meth:`setup` acquired."""

    def select_policy(self, nbytes: int) -> "CollectivePolicy":
        """The policy that carries a collective of ``nbytes``; may depend only on state that
        is identical on every rank."""
        return self

    # -- B200 additions ------------------------------------------------------------------------
    def stream_ordered(self, topology: "Topology") -> bool:
        """True when this policy only enqueues device work (never blocks the host), so the
        collective can start on the calling thread instead of the worker thread."""
        return False

    def fuses_average(self, topology: "Topology") -> bool:
        """True when ``all_reduce``/``reduce_scatter_tensor`` accept ``divide=`` and apply
        AVG inside the reducing kernel."""
        return False


# ---- fused execution ------------------------------------------------------------------------

class _Fused:
    """Mixin: run on ``topology.fabric`` when there is one and it can carry the call."""

    #: How the fabric's hierarchical all-reduce is shaped for this policy.
    fused_mode: ClassVar[str] = "auto"

    def stream_ordered(self, topology) -> bool:
        return topology.fabric is not None

    def fuses_average(self, topology) -> bool:
        return topology.fabric is not None

    def _fabric(self, topology, *tensors: torch.Tensor, op: str = "sum"):
        fabric = topology.fabric
        if fabric is None or not fabric.supports(tensors, op):
            return None
        return fabric


# ---- the policies -----------------------------------------------------------------------------

class NativeOnly(_Fused, CollectivePolicy):
    """One collective on the only island: the fused kernel on a box, else NCCL or Gloo."""

    name = "native-only"
    reduce_ops = _ALL_OPS

    @classmethod
    def applies_to(cls, layout):
        return not layout.needs_bridge

    def all_reduce(self, tensor, topology, op="sum", divide=None):
        fabric = self._fabric(topology, tensor, op=op)
        if fabric is not None:
            fabric.all_reduce(tensor, op=op, divide=divide)
            return
        topology.island_group.all_reduce(tensor, op)
        if divide:
            tensor.div_(divide)

    def broadcast(self, tensor, src, topology):
        fabric = self._fabric(topology, tensor)
        if fabric is not None:
            fabric.broadcast(tensor, src)
        else:
            topology.island_group.broadcast(tensor, src)

    def all_gather_into_tensor(self, output, input, topology):  # noqa: A002
        fabric = self._fabric(topology, output, input)
        if fabric is not None:
            fabric.all_gather(output, input)
        else:
            topology.island_group.all_gather_into(output, input)

    def reduce_scatter_tensor(self, output, input, topology, divide=None):  # noqa: A002
        fabric = self._fabric(topology, output, input)
        if fabric is not None:
            fabric.reduce_scatter(output, input, divide=divide)
            return
        topology.island_group.reduce_scatter_into(output, input)
        if divide:
            output.div_(divide)


class FlatGloo(CollectivePolicy):
    """Every rank stages to host memory and uses the Gloo group of all members.  No
    islands, no leaders, no bridge: the oracle the other policies are tested against."""

    name = "flat-gloo"
    reduce_ops = _ALL_OPS

    @classmethod
    def applies_to(cls, layout):
        return True

    def all_reduce(self, tensor, topology, op="sum"):
        host = _stage_to_host(tensor)
        topology.world_group.all_reduce(host, op)
        if host is not tensor:
            tensor.copy_(host)

    def broadcast(self, tensor, src, topology):
        host = _stage_to_host(tensor)
        topology.world_group.broadcast(host, src)
        if host is not tensor:
            tensor.copy_(host)

    def all_gather_into_tensor(self, output, input, topology):  # noqa: A002
        received = _host_like(output)
        topology.world_group.all_gather_into(received, _stage_to_host(input))
        if received.data_ptr() != output.data_ptr():
            output.copy_(received)

    def reduce_scatter_tensor(self, output, input, topology):  # noqa: A002
        received = _host_like(output)
        topology.world_group.reduce_scatter_into(received, _stage_to_host(input))
        if received.data_ptr() != output.data_ptr():
            output.copy_(received)


class ReduceBridgeBroadcast(_Fused, CollectivePolicy):
    """Reduce in each island, combine the island results over the bridge, broadcast back.

    Composed execution: ``reduce`` onto the leader, the leaders' bridge step (host-staged
    unless the transport takes device tensors; pinned with ``GPUBRIDGE_PINNED_STAGING``;
    compressed with ``GPUBRIDGE_BRIDGE_COMPRESSION``), ``broadcast`` from the leader.
    all_gather: island gather, every leader broadcasts its island's rows in turn, island
    broadcast.  reduce_scatter: island reduce, bridge all_reduce of the whole input, the
    leader scatters its members' slices.  Fused execution: see the module docstring.
    """

    name = "reduce-bridge-broadcast"
    reduce_ops = _ALL_OPS
    fused_mode = "auto"

    def __init__(self, compression: str | None = None) -> None:
        #: None follows ``GPUBRIDGE_BRIDGE_COMPRESSION``; "" switches it off; "bf16"/"fp8"
        #: pick a mode for this instance (a benchmark comparing modes in one job).
        self.compression = compression
        self.compressor: _compression.BridgeCompressor | None = None
        self.staging_buffer = None
        self.direct_bridge = False
        self._mode = ""
        self._fmt = "ref"

    # -- setup ---------------------------------------------------------------------------------
    def _setup_compression(self, topology, member: bool) -> None:
        mode = topology.bridge_compression if self.compression is None else self.compression
        self._mode = mode if topology.layout.needs_bridge else ""
        self._fmt = topology.codec_format
        self.compressor = (_compression.BridgeCompressor(mode, self._fmt)
                           if self._mode and member else None)

    def setup(self, topology):
        self._setup_compression(topology, member=topology.is_leader)
        if not (topology.layout.needs_bridge and topology.is_leader):
            return
        self.direct_bridge = (topology.device.type == "cuda"
                              and getattr(topology.bridge, "device_tensors", False))
        if topology.pinned_staging and not self.direct_bridge:
            self.staging_buffer = _staging.make_bridge_staging(topology.device)

    def close(self):
        if self.staging_buffer is not None:
            self.staging_buffer.close()
            self.staging_buffer = None
        self.compressor = None

    @classmethod
    def applies_to(cls, layout):
        return layout.needs_bridge

    def supported_reduce_ops(self, topology):
        assert topology.transport is not None
        return self.reduce_ops & topology.transport.reduce_ops

    def stream_ordered(self, topology):
        return topology.fabric is not None

    # -- helpers -------------------------------------------------------------------------------
    def _compresses(self, tensor, op) -> bool:
        return (bool(self._mode) and op == "sum" and tensor.numel() > 0
                and _compression.applies(self._mode, tensor.dtype))

    def _fused_compression(self, tensor, op):
        return (self._mode, self._fmt) if self._compresses(tensor, op) else None

    def _to_host(self, tensor):
        if self.direct_bridge:
            return tensor
        if self.staging_buffer is not None:
            return self.staging_buffer.to_host(tensor)
        return _stage_to_host(tensor)

    def _to_device(self, tensor, host):
        if host is tensor:
            return
        if self.staging_buffer is not None:
            self.staging_buffer.to_device(tensor, host)
        else:
            tensor.copy_(host)

    def _bridge_reduce(self, tensor, buffer, topology, op) -> None:
        """The leaders' step of a reduction; ``buffer`` owns the error-feedback residual."""
        if self._compresses(tensor, op):
            assert self.compressor is not None
            self.compressor.all_reduce(tensor.view(-1), _compression.buffer_key(buffer),
                                       topology.bridge, topology.layout.bridge_ranks,
                                       rank=topology.rank, direct=self.direct_bridge)
            return
        with phase("bridge"):
            host = self._to_host(tensor)
            topology.bridge.all_reduce(host, op)
            self._to_device(tensor, host)

    def _bridge_copy(self, tensor, topology, src_leader: int, receiving: bool) -> None:
        with phase("bridge"):
            host = self._to_host(tensor)
            topology.bridge.broadcast(host, src_leader)
            if receiving:
                self._to_device(tensor, host)

    # -- collectives -----------------------------------------------------------------------------
    def all_reduce(self, tensor, topology, op="sum", divide=None):
        fabric = self._fabric(topology, tensor, op=op)
        if fabric is not None:
            fabric.all_reduce(tensor, op=op, divide=divide, mode=self.fused_mode,
                              compression=self._fused_compression(tensor, op),
                              chunk_bytes=getattr(self, "chunk_bytes", None))
            return
        leader = topology.island.leader
        with phase("island-reduce"):
            topology.island_group.reduce(tensor, leader, op)
        if topology.is_leader:
            self._bridge_reduce(tensor, tensor, topology, op)
        with phase("island-broadcast"):
            topology.island_group.broadcast(tensor, leader)
        if divide:
            tensor.div_(divide)

    def broadcast(self, tensor, src, topology):
        fabric = self._fabric(topology, tensor)
        if fabric is not None:
            fabric.broadcast(tensor, src)
            return
        source = topology.layout.island_of(src)
        inside = topology.island == source
        if inside:
            with phase("island-broadcast"):
                topology.island_group.broadcast(tensor, src)
        if topology.is_leader:
            self._bridge_copy(tensor, topology, source.leader, receiving=not inside)
        if not inside:
            with phase("island-broadcast"):
                topology.island_group.broadcast(tensor, topology.island.leader)

    def all_gather_into_tensor(self, output, input, topology):  # noqa: A002
        fabric = self._fabric(topology, output, input)
        if fabric is not None:
            fabric.all_gather(output, input)
            return
        island, layout, n = topology.island, topology.layout, input.numel()
        rows = None
        with phase("island-gather"):
            if topology.is_leader:
                rows = torch.empty((len(island.ranks), n), dtype=input.dtype, device=input.device)
            topology.island_group.gather(input.reshape(-1),
                                         list(rows.unbind(0)) if rows is not None else None,
                                         island.leader)
        if topology.is_leader:
            with phase("bridge"):
                table = _host_like(output).view(layout.world_size, n)
                mine = _stage_to_host(rows)
                for other in layout.islands:       # the same order on every leader
                    part = mine if other == island else torch.empty(
                        (len(other.ranks), n), dtype=input.dtype)
                    topology.bridge.broadcast(part, other.leader)
                    table[[layout.index(r) for r in other.ranks]] = part
                if table.data_ptr() != output.data_ptr():
                    output.view(layout.world_size, n).copy_(table)
        with phase("island-broadcast"):
            topology.island_group.broadcast(output, island.leader)

    def reduce_scatter_tensor(self, output, input, topology, divide=None):  # noqa: A002
        fabric = self._fabric(topology, output, input)
        if fabric is not None:
            fabric.reduce_scatter(output, input, divide=divide,
                                  compression=self._fused_compression(input, "sum"))
            return
        island, layout = topology.island, topology.layout
        work = input.clone()                      # the input stays unmodified
        with phase("island-reduce"):
            topology.island_group.reduce(work, island.leader)
        if topology.is_leader:
            self._bridge_reduce(work, input, topology, "sum")
        with phase("island-scatter"):
            slices = work.view(layout.world_size, -1)
            topology.island_group.scatter(
                output.view(-1),
                [slices[layout.index(r)] for r in island.ranks] if topology.is_leader else None,
                island.leader)
        if divide:
            output.div_(divide)


class PipelinedReduceBridgeBroadcast(ReduceBridgeBroadcast):
    """reduce-bridge-broadcast with the bridge step cut into ``GPUBRIDGE_CHUNK_BYTES``
    chunks (default 4 MiB).

    Composed execution on GPUs: three pinned slots; the copy of chunk k+1 to the host, the
    bridge step of chunk k and the copy of chunk k-1 back run at the same time, ordered by
    events; the last copy back out of each slot is remembered across collectives.  Fused
    execution: the kernel walks the tensor in chunks of the same size, so the cross-island
    stage of chunk k overlaps the island stages of its neighbours.
    """

    name = "pipelined-reduce-bridge-broadcast"
    fused_mode = "chunked"
    SLOTS = 3
    DEFAULT_CHUNK_BYTES = 4 << 20

    def __init__(self, chunk_bytes: int | None = None, compression: str | None = None) -> None:
        super().__init__(compression)
        self.chunk_bytes = chunk_bytes
        self.staging = None
        self.copied_back: list[Any] = [None] * self.SLOTS
        self.recv_staging = None
        self.recv_back: list[Any] = []

    @classmethod
    def settings(cls):
        return {"chunk_bytes": chunk_bytes_setting(cls.DEFAULT_CHUNK_BYTES)}

    def setup(self, topology):
        if self.chunk_bytes is None:
            self.chunk_bytes = int(topology.policy_settings.get("chunk_bytes",
                                                                self.DEFAULT_CHUNK_BYTES))
        self._setup_compression(topology, member=topology.is_leader)
        if (topology.layout.needs_bridge and topology.is_leader and topology.fabric is None):
            self.staging = _staging.make_staging(topology.device, self.chunk_bytes, self.SLOTS)
            if self.compressor is not None:
                slots = self.SLOTS * (len(topology.layout.islands) - 1)
                self.recv_staging = _staging.make_staging(topology.device, self.chunk_bytes, slots)
                self.recv_back = [None] * slots

    def close(self):
        for staging in (self.staging, self.recv_staging):
            if staging is not None:
                staging.close()
        self.staging = self.recv_staging = None
        self.copied_back = [None] * self.SLOTS
        self.recv_back = []
        self.compressor = None

    def _bridge_reduce(self, tensor, buffer, topology, op):
        bridge = topology.bridge
        if self._compresses(tensor, op):
            self._compressed_pipeline(tensor, buffer, topology)
            return
        with phase("bridge"):
            self._pipeline(tensor, lambda host: bridge.all_reduce(host, op), send=True,
                           receive=True)

    def _bridge_copy(self, tensor, topology, src_leader, receiving):
        bridge = topology.bridge
        with phase("bridge"):
            self._pipeline(tensor, lambda host: bridge.broadcast(host, src_leader),
                           send=not receiving, receive=receiving)

    def _pipeline(self, tensor, step, *, send: bool, receive: bool) -> None:
        """``step`` on every chunk's host slot; copies of neighbouring chunks overlap it."""
        staging, slots = self.staging, self.SLOTS
        flat = tensor.view(-1)
        width = max(1, self.chunk_bytes // tensor.element_size())
        chunks = [flat[lo:lo + width] for lo in range(0, flat.numel(), width)]
        out_events: list[Any] = [None] * len(chunks)
        last_back = None

        def copy_out(k: int) -> None:
            slot = staging.slot(k % slots, chunks[k])
            out_events[k] = staging.to_host(slot, chunks[k], self.copied_back[k % slots])

        staging.begin(tensor)
        if send and chunks:
            copy_out(0)
        for k, chunk in enumerate(chunks):
            if send and k + 1 < len(chunks):
                copy_out(k + 1)
            host = staging.slot(k % slots, chunk)
            # Before the bridge touches the slot: its data has arrived (send) or the last
            # copy back out of it has finished (receive only).
            staging.wait_host(out_events[k] if send else self.copied_back[k % slots])
            step(host)
            if receive:
                self.copied_back[k % slots] = last_back = staging.to_device(chunk, host)
        staging.end(last_back)

    def _compressed_pipeline(self, tensor, buffer, topology) -> None:
        """Quantise the whole island result once, exchange the payloads chunk by chunk
        through the host slots, dequantise once."""
        bridge, members = topology.bridge, topology.layout.bridge_ranks
        me = members.index(topology.rank)
        flat = tensor.view(-1)
        rows = self.compressor.compress(flat, _compression.buffer_key(buffer), members, me)
        with phase("bridge"):
            self._exchange(rows, me, members, bridge)
        self.compressor.decompress(rows, flat)

    def _exchange(self, rows, me, members, bridge) -> None:
        staging, recv, slots = self.staging, self.recv_staging, self.SLOTS
        width = rows.shape[1]
        cuts = [(lo, min(lo + self.chunk_bytes, width)) for lo in range(0, width, self.chunk_bytes)]
        others = [i for i in range(len(members)) if i != me]
        mine = rows[me]
        out_events: list[Any] = [None] * len(cuts)
        last_back = None

        def copy_out(k: int) -> None:
            lo, hi = cuts[k]
            slot = staging.slot(k % slots, mine[lo:hi])
            out_events[k] = staging.to_host(slot, mine[lo:hi], self.copied_back[k % slots])

        staging.begin(rows)
        recv.begin(rows)
        if cuts:
            copy_out(0)
        for k, (lo, hi) in enumerate(cuts):
            if k + 1 < len(cuts):
                copy_out(k + 1)
            hosts: dict[int, torch.Tensor] = {}
            for j, i in enumerate(others):
                index = (k % slots) * len(others) + j
                recv.wait_host(self.recv_back[index])   # the bridge is about to overwrite it
                hosts[i] = recv.slot(index, rows[i, lo:hi])
            staging.wait_host(out_events[k])
            hosts[me] = staging.slot(k % slots, mine[lo:hi])
            for i, src in enumerate(members):
                bridge.broadcast(hosts[i], src)
            for j, i in enumerate(others):
                index = (k % slots) * len(others) + j
                self.recv_back[index] = last_back = recv.to_device(rows[i, lo:hi], hosts[i])
        recv.end(last_back)


_link_setups: dict[str, int] = {}      # topology context name -> sharded-bridge set-ups so far


class ShardedBridge(ReduceBridgeBroadcast):
    """k ranks per island share the bridge step, one stripe each (k = smallest island).

    Rank j of every island joins bridge link j (link 0 is the leaders' bridge).  all_reduce
    on the tensor padded to k stripes: the island leaves its reduction of stripe j on its
    rank j (one reduce_scatter when the island has exactly k ranks, else k reduces); rank j
    of every island all_reduces stripe j over link j; the island reassembles (all_gather or
    k broadcasts).  This is the two-level all-reduce with islands in place of nodes.  Fused
    execution is the same shape inside one kernel: every stripe owner is the "leader" of its
    stripe and the stripes cross the islands at the same time over NVLink.
    """

    name = "sharded-bridge"
    fused_mode = "striped"

    def __init__(self, compression: str | None = None) -> None:
        super().__init__(compression)
        self.k = 1
        self.index = 0
        self.link = None
        self.link_members: tuple[int, ...] = ()
        self._created: list["BridgeTransport"] = []

    def setup(self, topology):
        islands = topology.layout.islands
        self.k = min(len(i.ranks) for i in islands)
        self.index = topology.island.ranks.index(topology.rank)
        self._setup_compression(topology, member=self.index < self.k)
        if topology.fabric is not None or not topology.layout.needs_bridge:
            return
        groups = [sorted(i.ranks[j] for i in islands) for j in range(1, self.k)]
        links: list = []
        if groups:
            # A second instance of this policy on the same topology (a benchmark racing
            # policies, an auto-tuned policy's candidates) must not meet the first one's store
            # keys: the count of set-ups - the same on every rank, set-up being collective -
            # is part of the links' names.
            context = topology.context
            count = _link_setups[context.name] = _link_setups.get(context.name, 0) + 1
            if count > 1:
                context = dataclasses.replace(context, name=f"{context.name}.setup{count}")
            links = topology.transport.create_groups(groups, timeout=topology.timeout,
                                                     context=context)
            for ranks, link in zip(groups, links):
                if (link is not None) != (topology.rank in ranks):
                    raise RuntimeError(
                        f"{topology.transport.__name__}.create_groups() must return a transport "
                        f"exactly on each group's members; rank {topology.rank} got {link!r} "
                        f"for {ranks}")
        self._created = [link for link in links if link is not None]
        if self.index == 0:
            self.link = topology.bridge
        elif self.index < self.k:
            self.link = links[self.index - 1]
        if self.index < self.k:
            self.link_members = tuple(sorted(i.ranks[self.index] for i in islands))

    def close(self):
        for link in self._created:
            link.close()
        self._created, self.link = [], None
        self.compressor = None

    def _stripes(self, tensor):
        """``tensor`` flattened, and a buffer of k equal stripes holding it (itself when it
        divides evenly; padding is zero, reduced only with padding, never copied back)."""
        flat = tensor.view(-1)
        size = -(-flat.numel() // self.k) * self.k
        if size == flat.numel():
            return flat, flat
        padded = torch.zeros(size, dtype=flat.dtype, device=flat.device)
        padded[:flat.numel()].copy_(flat)
        return flat, padded

    def _reassemble(self, padded, mine, topology) -> None:
        island, group = topology.island, topology.island_group
        if len(island.ranks) == self.k:
            with phase("island-all-gather"):
                group.all_gather_into(padded, mine)
            return
        stripes = padded.view(self.k, -1)
        with phase("island-broadcast"):
            for j in range(self.k):
                group.broadcast(stripes[j], island.ranks[j])

    def all_reduce(self, tensor, topology, op="sum", divide=None):
        fabric = self._fabric(topology, tensor, op=op)
        if fabric is not None:
            fabric.all_reduce(tensor, op=op, divide=divide, mode="striped",
                              compression=self._fused_compression(tensor, op))
            return
        flat, padded = self._stripes(tensor)
        stripes = padded.view(self.k, -1)
        island, group = topology.island, topology.island_group
        mine = None
        if len(island.ranks) == self.k:
            with phase("island-reduce-scatter"):
                mine = torch.empty_like(stripes[0])
                group.reduce_scatter_into(mine, padded, op)
        else:
            with phase("island-reduce"):
                for j in range(self.k):
                    group.reduce(stripes[j], island.ranks[j], op)
            if self.index < self.k:
                mine = stripes[self.index]
        if self.link is not None:
            if self._compresses(mine, op):
                self.compressor.all_reduce(mine, _compression.buffer_key(tensor, self.index),
                                           self.link, self.link_members, rank=topology.rank)
            else:
                with phase("bridge"):
                    host = _stage_to_host(mine)
                    self.link.all_reduce(host, op)
                    if host is not mine:
                        mine.copy_(host)
        self._reassemble(padded, mine, topology)
        if padded is not flat:
            flat.copy_(padded[:flat.numel()])
        if divide:
            tensor.div_(divide)

    def broadcast(self, tensor, src, topology):
        fabric = self._fabric(topology, tensor)
        if fabric is not None:
            fabric.broadcast(tensor, src)
            return
        source = topology.layout.island_of(src)
        inside = topology.island == source
        if inside:
            with phase("island-broadcast"):
                topology.island_group.broadcast(tensor, src)
        flat, padded = self._stripes(tensor)
        stripes = padded.view(self.k, -1)
        mine = None
        if self.index < self.k:
            exact = len(topology.island.ranks) == self.k
            mine = (torch.empty_like(stripes[0]) if exact and not inside
                    else stripes[self.index])
        if self.link is not None:
            with phase("bridge"):
                host = _stage_to_host(mine)
                self.link.broadcast(host, source.ranks[self.index])
                if not inside and host is not mine:
                    mine.copy_(host)
        if not inside:
            self._reassemble(padded, mine, topology)
            if padded is not flat:
                flat.copy_(padded[:flat.numel()])


class AutoTuned(CollectivePolicy):
    """A policy per message size, from a thresholds file measured on the cluster
    (``GPUBRIDGE_THRESHOLDS``; written by ``bench_all_reduce.py --write-thresholds``).  Without
    the variable every size gets what ``auto`` picks.  The rules are part of the policy's
    settings, so discovery refuses ranks that loaded different files."""

    name = "auto-tuned"
    reduce_ops = _ALL_OPS

    def __init__(self) -> None:
        self.rules: list[tuple[int | None, CollectivePolicy]] = []

    @classmethod
    def applies_to(cls, layout):
        return True

    @classmethod
    def settings(cls):
        path = os.environ.get(THRESHOLDS_ENV, "").strip()
        chunk = chunk_bytes_setting(PipelinedReduceBridgeBroadcast.DEFAULT_CHUNK_BYTES)
        if not path:
            return {"rules": [{"max_bytes": None, "policy": AUTO}], "chunk_bytes": chunk}
        return load_thresholds(path, chunk)

    def setup(self, topology):
        settings = topology.policy_settings
        for rule in settings["rules"]:
            try:
                cls = choose_policy(resolve_policy(rule["policy"]), topology.layout)
            except RuntimeError as exc:
                raise RuntimeError(f"{THRESHOLDS_ENV}: the rule for sizes up to "
                                   f"{rule['max_bytes']} bytes can't be used here. {exc}") from None
            policy = (cls(chunk_bytes=settings["chunk_bytes"])
                      if issubclass(cls, PipelinedReduceBridgeBroadcast) else cls())
            policy.setup(topology)
            self.rules.append((rule["max_bytes"], policy))

    def close(self):
        for _, policy in self.rules:
            policy.close()

    def select_policy(self, nbytes):
        for max_bytes, policy in self.rules:
            if max_bytes is None or nbytes <= max_bytes:
                return policy.select_policy(nbytes)
        raise AssertionError("the last thresholds rule covers every size")

    def supported_reduce_ops(self, topology):
        ops = self.reduce_ops
        for _, policy in self.rules:
            ops &= policy.supported_reduce_ops(topology)
        return ops

    def stream_ordered(self, topology):
        return all(p.stream_ordered(topology) for _, p in self.rules)

    def all_reduce(self, tensor, topology, op="sum"):
        self.select_policy(tensor.nbytes).all_reduce(tensor, topology, op)

    def broadcast(self, tensor, src, topology):
        self.select_policy(tensor.nbytes).broadcast(tensor, src, topology)

    def all_gather_into_tensor(self, output, input, topology):  # noqa: A002
        self.select_policy(output.nbytes).all_gather_into_tensor(output, input, topology)

    def reduce_scatter_tensor(self, output, input, topology):  # noqa: A002
        self.select_policy(input.nbytes).reduce_scatter_tensor(output, input, topology)


THRESHOLDS_FORMAT = 1


def load_thresholds(path: str, chunk_bytes: int) -> dict[str, Any]:
    """Read and check a thresholds file (format 1:
    ``{"gpubridge_thresholds": 1, "rules": [{"max_bytes": N|null, "policy": name}, ...],
    "chunk_bytes": N}``); every error names the variable and what is wrong."""
    where = f"{THRESHOLDS_ENV}={path!r}"
    try:
        with open(path) as fh:
            data = json.load(fh)
    except OSError as exc:
        raise ValueError(f"{where}: can't read it ({exc.strerror or exc})") from None
    except json.JSONDecodeError as exc:
        raise ValueError(f"{where}: not valid JSON ({exc})") from None
    if not isinstance(data, dict) or data.get("gpubridge_thresholds") != THRESHOLDS_FORMAT:
        raise ValueError(f"{where}: not a gpubridge thresholds file (format {THRESHOLDS_FORMAT}); "
                         "write one with bench_all_reduce.py --write-thresholds")
    rules = data.get("rules")
    if not isinstance(rules, list) or not rules:
        raise ValueError(f"{where}: needs a non-empty list of rules")
    checked, previous = [], -1
    for i, rule in enumerate(rules):
        name, limit = (rule.get("policy"), rule.get("max_bytes")) if isinstance(rule, dict) \
            else (None, None)
        last = i == len(rules) - 1
        if name == AutoTuned.name or (name != AUTO and name not in _POLICIES):
            known = ", ".join([AUTO, *sorted(n for n in _POLICIES if n != AutoTuned.name)])
            raise ValueError(f"{where}: rule {i} names policy {name!r}; known: {known}")
        if last and limit is not None:
            raise ValueError(f"{where}: the last rule must cover every size (max_bytes null)")
        if not last and (not isinstance(limit, int) or isinstance(limit, bool)
                         or limit <= previous):
            raise ValueError(f"{where}: rule {i} needs an integer max_bytes larger than the "
                             "previous rule's")
        previous = limit if limit is not None else previous
        checked.append({"max_bytes": limit, "policy": name})
    chunk = data.get("chunk_bytes", chunk_bytes)
    if not isinstance(chunk, int) or chunk < 8 or chunk % 8:
        raise ValueError(f"{where}: chunk_bytes must be a positive multiple of 8")
    return {"rules": checked, "chunk_bytes": chunk}


def write_thresholds(path: str, rules: list[dict[str, Any]], chunk_bytes: int) -> None:
    """Write a format-1 thresholds file."""
    with open(path, "w") as fh:
        json.dump({"gpubridge_thresholds": THRESHOLDS_FORMAT, "rules": rules,
                   "chunk_bytes": chunk_bytes}, fh, indent=1)


DEFAULT_POLICY = AUTO

_POLICIES: dict[str, type[CollectivePolicy]] = {
    cls.name: cls for cls in (ReduceBridgeBroadcast, NativeOnly, FlatGloo,
                              PipelinedReduceBridgeBroadcast, ShardedBridge, AutoTuned)}


def register_policy(policy: type[CollectivePolicy]) -> type[CollectivePolicy]:
    """Make ``policy`` selectable by name (usable as a class decorator)."""
    if not (isinstance(policy, type) and issubclass(policy, CollectivePolicy)):
        raise TypeError(f"expected a CollectivePolicy subclass, got {policy!r}")
    if policy.name == AUTO:
        raise ValueError(f"{AUTO!r} is reserved for automatic selection")
    existing = _POLICIES.get(policy.name)
    if existing is not None and existing is not policy:
        raise ValueError(f"a different policy is already registered as {policy.name!r}")
    _POLICIES[policy.name] = policy
    return policy


def resolve_policy(policy):
    """``"auto"``, a registered name or a policy class -> ``"auto"`` or the class."""
    if isinstance(policy, str):
        if policy == AUTO:
            return AUTO
        try:
            return _POLICIES[policy]
        except KeyError:
            known = ", ".join([AUTO, *sorted(_POLICIES)])
            raise ValueError(f"unknown collective policy {policy!r}; known: {known}") from None
    if isinstance(policy, type) and issubclass(policy, CollectivePolicy):
        return policy
    raise TypeError(f"policy must be a policy name or CollectivePolicy subclass, got {policy!r}")


def implements(policy, fn: str) -> bool:
    cls = policy if isinstance(policy, type) else type(policy)
    return getattr(cls, fn) is not getattr(CollectivePolicy, fn)


def policies_implementing(fn: str, layout) -> list[str]:
    return sorted(n for n, c in _POLICIES.items() if c.applies_to(layout) and implements(c, fn))


def policy_name(policy) -> str:
    return policy if isinstance(policy, str) else policy.name


def choose_policy(policy, layout) -> type[CollectivePolicy]:
    """The class to run on ``layout``; ``auto`` never picks an opt-in policy."""
    if isinstance(policy, str):
        assert policy == AUTO
        return ReduceBridgeBroadcast if layout.needs_bridge else NativeOnly
    if not policy.applies_to(layout):
        n = len(layout.islands)
        usable = ", ".join([AUTO, *sorted(k for k, c in _POLICIES.items() if c.applies_to(layout))])
        raise RuntimeError(f"Collective policy {policy.name!r} doesn't apply to this cluster "
                           f"({n} island{'s' if n != 1 else ''}). Policies that do: {usable}.")
    return policy
