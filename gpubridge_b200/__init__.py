"""gpubridge-b200: a Blackwell-native hierarchical collective backend for PyTorch.

Ranks form **islands** (one label each; on one 8xB200 box islands are made the way the
reference's split tests make them), an island's lowest rank is its **leader**, the leaders
are joined by the **bridge**, and a **collective policy** composes group-wide collectives
from island steps and the bridge step.  On a GPU box the whole composition is one
hand-written sm_100a kernel over NVLink peer memory; on CPU (simulation mode) and across
nodes it is composed from Gloo/NCCL collectives and a host-staged bridge transport.

Public surface (the reference's: src/gpubridge/__init__.py:72-221): ``init``, ``destroy``,
``all_reduce``, ``broadcast``, ``all_gather_into_tensor``, ``reduce_scatter_tensor``,
``barrier``, ``Work`` handles, ``ddp_comm_hook``, observers and ``in_flight``, policy and
transport registries, and the ``torch.distributed`` backend ``backend="gpubridge"``.
"""
from __future__ import annotations

from datetime import timedelta
from typing import Any

import torch.distributed as dist
from torch.distributed import ReduceOp

from gpubridge_b200 import observe as _observe
from gpubridge_b200 import topology as _topology
from gpubridge_b200 import work as _work
from gpubridge_b200.collectives import (SUPPORTED_DTYPES, all_gather_into_tensor, all_reduce,
                                        barrier, broadcast, reduce_scatter_tensor)
from gpubridge_b200.compression import reset_error_feedback
from gpubridge_b200.config import CPU_BACKEND
from gpubridge_b200.ddp import ddp_comm_hook
from gpubridge_b200.detect import Probe, probe
from gpubridge_b200.observe import (CollectiveObserver, CollectiveRecord, InFlight, Mark, Phase,
                                    add_observer, elapsed_ms, in_flight, remove_observer)
from gpubridge_b200.policies import (DEFAULT_POLICY, CollectivePolicy, register_policy,
                                     resolve_policy)
from gpubridge_b200.split_test import SplitTestWarning
from gpubridge_b200.topology import (Island, Layout, PeerInfo, Topology, get_topology,
                                     is_initialized)
from gpubridge_b200.transport import (DEFAULT_TRANSPORT, BridgeTransport, GlooTransport,
                                      LinkContext, NvlinkTransport, register_transport,
                                      resolve_transport)
from gpubridge_b200.work import Work
from gpubridge_b200 import torch_backend as _torch_backend

_torch_backend.register()
batch_isend_irecv = _torch_backend.batch_isend_irecv

__version__ = "0.1.0"

__all__ = [
    "batch_isend_irecv", "BridgeTransport", "CollectiveObserver", "CollectivePolicy",
    "CollectiveRecord", "GlooTransport", "InFlight", "Island", "Layout", "LinkContext", "Mark",
    "NvlinkTransport", "PeerInfo", "Phase", "Probe", "ReduceOp", "SplitTestWarning",
    "SUPPORTED_DTYPES", "Topology", "Work", "add_observer", "all_gather_into_tensor",
    "all_reduce", "barrier", "broadcast", "ddp_comm_hook", "destroy", "elapsed_ms",
    "get_topology", "in_flight", "init", "is_initialized", "probe", "reduce_scatter_tensor",
    "register_policy", "register_transport", "remove_observer", "reset_error_feedback",
]

_generation = 0


def init(init_method: str | None = None, *, rank: int | None = None,
         world_size: int | None = None, timeout: timedelta | None = None,
         bridge: "str | type[BridgeTransport] | None" = None,
         policy: "str | type[CollectivePolicy]" = DEFAULT_POLICY) -> Topology:
    """Join the job and build this rank's topology.  Call once on every rank.

    The arguments mirror ``torch.distributed.init_process_group``; with none given the
    ``env://`` variables of torchrun are used.  The library owns the default process group
    (a Gloo group of every rank); discovery, the island communicators, the bridge and - on
    a GPU box - the NVLink fabric are bootstrapped over that group's store.  ``bridge``
    defaults to ``"nvlink"`` for GPU ranks and ``"gloo"`` for CPU simulation.

    Raises ``RuntimeError`` when already initialised, when any rank reported a problem (no
    vendor, no GPU, no NCCL), when ranks disagree on mode, bridge, policy or settings, or
    when the policy doesn't fit the layout; ``ValueError`` for unknown names or bad
    ``GPUBRIDGE_*`` values.
    """
    global _generation
    if is_initialized():
        raise RuntimeError("gpubridge is already initialized")
    if dist.is_initialized():
        raise RuntimeError("torch.distributed is already initialized; gpubridge.init() creates "
                           "the default process group itself")
    from gpubridge_b200.config import is_simulated
    if bridge is None:
        bridge = DEFAULT_TRANSPORT if is_simulated() else NvlinkTransport.name
    transport = resolve_transport(bridge)
    chosen = resolve_policy(policy)
    local, cfg = _topology.describe_local(transport.name, chosen)
    kwargs: dict[str, Any] = {}
    if rank is not None:
        kwargs["rank"] = rank
    if world_size is not None:
        kwargs["world_size"] = world_size
    if timeout is not None:
        kwargs["timeout"] = timeout
    dist.init_process_group(backend=CPU_BACKEND, init_method=init_method, **kwargs)
    try:
        store = dist.distributed_c10d._get_default_store()
        _generation += 1
        topology = _topology.build_topology(
            store, dist.get_rank(), dist.get_world_size(), local, cfg, transport=transport,
            policy=chosen, timeout=timeout, name=f"init{_generation}")
    except BaseException:
        dist.destroy_process_group()
        raise
    _work.shutdown()
    _observe._reset()
    _topology._set_topology(topology)
    return topology


def destroy() -> None:
    """Run queued async collectives, then release every group :func:`init` created."""
    if not is_initialized():
        return
    try:
        _release()
    finally:
        dist.destroy_process_group()


def _release(drain: bool = True) -> None:
    topology = get_topology()
    try:
        if drain:
            _work.shutdown()
        else:
            _work.abandon()
    finally:
        _topology._set_topology(None)
        _observe._reset()
    _topology.close_topology(topology)
