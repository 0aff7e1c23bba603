"""Bridge transports: what joins the island leaders.

On one NVSwitch box the bridge is NVLink itself (``nvlink``: the fused kernels move the
leaders' data, this class only carries the name, the reductions and a device fallback).
The host-staged transports of the reference survive as the cross-node fallback and as
what CPU simulation runs: ``gloo`` (a Gloo group of the leaders; reference:
src/gpubridge/transport.py:127-153) and ``multitcp`` (native multi-stream TCP worker,
:mod:`gpubridge_b200.multitcp`).  ``ucx`` (:mod:`gpubridge_b200.ucx`: a worker compiled at first
use against the machine's UCX) and ``verbs`` (:mod:`gpubridge_b200.rdma`) load when what they need
is there and otherwise say, on every rank alike, what is missing, as the reference's loaders do
(src/gpubridge/ucx/__init__.py:45-46).
"""
from __future__ import annotations

import abc
import importlib
from collections.abc import Sequence
from dataclasses import dataclass
from datetime import timedelta
from typing import Any, ClassVar

import torch

from gpubridge_b200.groups import Comm, make_comm


@dataclass(frozen=True)
class LinkContext:
    """What a transport needs to set a link up: the job's store, this process's global
    rank, and a name that is unique per link and equal on all of its members."""

    store: Any
    rank: int
    name: str
    device: torch.device = torch.device("cpu")


class BridgeTransport(abc.ABC):
    """Moves tensors between the members of one bridge link.  One instance per member."""

    name: ClassVar[str]
    #: Always "sum"; "max"/"min" when listed.
    reduce_ops: ClassVar[frozenset[str]] = frozenset({"sum"})
    #: True when all_reduce/broadcast take device tensors and order them on the current
    #: stream themselves, so policies skip host staging.
    device_tensors: ClassVar[bool] = False

    @classmethod
    @abc.abstractmethod
    def create(cls, ranks: Sequence[int], *, context: LinkContext,
               timeout: timedelta | None = None) -> "BridgeTransport | None":
        """Build the link over ``ranks`` (global).  Called by every process that builds the
        topology; returns an instance exactly on the members."""

    @classmethod
    def create_groups(cls, groups: Sequence[Sequence[int]], *, context: LinkContext,
                      timeout: timedelta | None = None) -> list["BridgeTransport | None"]:
        """One link per entry of ``groups`` (the sharded policy's extra links)."""
        return [cls.create(ranks, timeout=timeout,
                           context=LinkContext(context.store, context.rank,
                                               f"{context.name}.{i}", context.device))
                for i, ranks in enumerate(groups)]

    @abc.abstractmethod
    def all_reduce(self, tensor: torch.Tensor, op: str = "sum") -> None:
        """Reduce a contiguous tensor over the link's members, in place."""

    @abc.abstractmethod
    def broadcast(self, tensor: torch.Tensor, src: int) -> None:
        """Copy from member ``src`` (a global rank), in place."""

    def close(self) -> None:  # noqa: B027 - optional
        """Release what :meth:`create` acquired."""

    @classmethod
    def create_p2p(cls, group: Comm, *, store=None, timeout=None):
        """An all-member point-to-point link for cross-island send/recv; optional."""
        raise NotImplementedError(f"bridge transport {cls.name!r} has no point-to-point link")


class GlooTransport(BridgeTransport):
    """A Gloo group of the link's members; carries host tensors."""

    name = "gloo"
    reduce_ops = frozenset({"sum", "max", "min"})

    def __init__(self, group: Comm) -> None:
        self.group = group

    @classmethod
    def create(cls, ranks, *, context, timeout=None):
        group = make_comm(context.store, f"bridge.{context.name}", ranks, context.rank, "gloo",
                          timeout)
        return cls(group) if group is not None else None

    def all_reduce(self, tensor, op="sum"):
        self.group.all_reduce(tensor, op)

    def broadcast(self, tensor, src):
        self.group.broadcast(tensor, src)

    def close(self):
        self.group.close()

    @classmethod
    def create_p2p(cls, group, *, store=None, timeout=None):
        from gpubridge_b200.p2p import GlooLink
        return GlooLink(group)


class NvlinkTransport(GlooTransport):
    """The bridge of a single NVSwitch box.

    The fused policies never call it: the leaders' exchange happens inside the collective
    kernel over peer memory.  It still is a complete transport (an NCCL group of the
    leaders, device tensors in and out) for policies that compose collectives step by step,
    e.g. a user-registered one.
    """

    name = "nvlink"
    device_tensors = True

    @classmethod
    def create(cls, ranks, *, context, timeout=None):
        kind = "nccl" if context.device.type == "cuda" else "gloo"
        group = make_comm(context.store, f"bridge.{context.name}", ranks, context.rank, kind,
                          timeout, context.device)
        return cls(group) if group is not None else None


DEFAULT_TRANSPORT = GlooTransport.name
_TRANSPORTS: dict[str, type[BridgeTransport]] = {
    GlooTransport.name: GlooTransport, NvlinkTransport.name: NvlinkTransport}
#: Opt-in transports, imported at first use.
_BUILT_IN = {"multitcp": "gpubridge_b200.multitcp", "ucx": "gpubridge_b200.ucx.transport",
             "verbs": "gpubridge_b200.rdma"}


def _load_built_in(name: str) -> None:
    module = _BUILT_IN.get(name)
    if module is None or name in _TRANSPORTS:
        return
    try:
        loaded = importlib.import_module(module)
        if hasattr(loaded, "load"):
            loaded.load(name)
    except ImportError as exc:
        raise ValueError(f"bridge transport {name!r} can't be loaded: {exc}") from exc


def register_transport(transport: type[BridgeTransport]) -> type[BridgeTransport]:
    """Make ``transport`` selectable by name (usable as a class decorator)."""
    if not (isinstance(transport, type) and issubclass(transport, BridgeTransport)):
        raise TypeError(f"expected a BridgeTransport subclass, got {transport!r}")
    existing = _TRANSPORTS.get(transport.name)
    if existing is not None and existing is not transport:
        raise ValueError(f"a different transport is already registered as {transport.name!r}")
    _TRANSPORTS[transport.name] = transport
    return transport


def resolve_transport(bridge: str | type[BridgeTransport]) -> type[BridgeTransport]:
    if isinstance(bridge, str):
        _load_built_in(bridge)
        try:
            return _TRANSPORTS[bridge]
        except KeyError:
            known = ", ".join(sorted({*_TRANSPORTS, *_BUILT_IN}))
            raise ValueError(f"unknown bridge transport {bridge!r}; known: {known}") from None
    if isinstance(bridge, type) and issubclass(bridge, BridgeTransport):
        return bridge
    raise TypeError(f"bridge must be a transport name or BridgeTransport subclass, got {bridge!r}")
