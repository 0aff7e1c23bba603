"""Discovery, islands, leaders and the bridge.

The model is the reference's (src/gpubridge/topology.py:42-444): ranks are grouped into
**islands** by label, an island's lowest rank is its **leader**, the leaders form the
**bridge**; every rank describes itself in a :class:`PeerInfo` (whose wire dictionary keeps
the reference's field names), problems are *recorded* and then raised with one text on
every rank, and every setting that changes how many messages a collective sends must agree.

What differs is how groups come to exist: everything is bootstrapped over the job's c10d
``Store`` (:mod:`gpubridge_b200.groups`).  Discovery is a keyed exchange on the store, each
communicator is constructed by its members only, and a subgroup (a ``DeviceMesh``
dimension, ``dist.new_group``) builds its own topology the same way under its own store
prefix - no job-wide ``new_group`` ordering, no patching of torch's private group naming.

On GPUs, when every member sits on one NVSwitch box, the topology also carries a
**fabric** (:mod:`gpubridge_b200.ops.fabric`): symmetric buffers mapped into every peer,
which the fused collective kernels run on.
"""
from __future__ import annotations

import json
import time
import warnings
from collections.abc import Sequence
from dataclasses import asdict, dataclass, field
from datetime import timedelta
from functools import cached_property
from typing import Any, cast

import torch
import torch.distributed as dist

from gpubridge_b200 import config as _config
from gpubridge_b200.config import (BRIDGE_COMPRESSION_ENV, CPU_ONLY_ENV, GPU_BACKEND,
                                   ISLANDS_ENV, PINNED_STAGING_ENV, SPLIT_TEST_ENV, VENDOR_ENV,
                                   Config)
from gpubridge_b200.detect import Probe, detect_vendor, probe
from gpubridge_b200.groups import DEFAULT_TIMEOUT, Comm, make_comm
from gpubridge_b200.policies import AUTO, CollectivePolicy, choose_policy, policy_name
from gpubridge_b200.split_test import SplitTestWarning, banner, island_labels, split_labels
from gpubridge_b200.transport import BridgeTransport, LinkContext


@dataclass(frozen=True)
class Island:
    """The ranks sharing one label; they share a native communicator."""

    vendor: str
    ranks: tuple[int, ...]

    @property
    def leader(self) -> int:
        return self.ranks[0]


@dataclass(frozen=True)
class Layout:
    """How a group's members split into islands.  Pure data, equal on every member."""

    vendors: tuple[str, ...]
    islands: tuple[Island, ...]
    ranks: tuple[int, ...] = ()
    """A subgroup's members (global ranks, ascending); empty for the world."""

    @property
    def world_size(self) -> int:
        return len(self.vendors)

    @property
    def members(self) -> tuple[int, ...]:
        return self.ranks or tuple(range(len(self.vendors)))

    def index(self, rank: int) -> int:
        """A member's position in the group: its row of an all_gather."""
        return self.ranks.index(rank) if self.ranks else rank

    @property
    def bridge_ranks(self) -> tuple[int, ...]:
        return tuple(i.leader for i in self.islands)

    @property
    def needs_bridge(self) -> bool:
        return len(self.islands) > 1

    def island_of(self, rank: int) -> Island:
        label = self.vendors[self.index(rank)]
        for island in self.islands:
            if island.vendor == label:
                return island
        raise KeyError(rank)

    def island_index(self, rank: int) -> int:
        return self.islands.index(self.island_of(rank))


def plan_topology(vendors: Sequence[str], ranks: Sequence[int] = ()) -> Layout:
    """Islands (ordered by leader) from each member's label.  A pure function, so every
    rank that sees the same labels plans the same islands, leaders and bridge."""
    if not vendors:
        raise ValueError("cannot plan a topology for zero ranks")
    if ranks and (len(ranks) != len(vendors) or list(ranks) != sorted(set(ranks))):
        raise ValueError(f"a subgroup's ranks must be distinct and ascending, got {list(ranks)}")
    members = tuple(ranks) or tuple(range(len(vendors)))
    grouped: dict[str, list[int]] = {}
    for rank, label in zip(members, vendors):
        grouped.setdefault(label, []).append(rank)
    islands = sorted((Island(label, tuple(rs)) for label, rs in grouped.items()),
                     key=lambda island: island.leader)
    return Layout(tuple(vendors), tuple(islands), tuple(ranks))


@dataclass(frozen=True)
class PeerInfo:
    """What a rank reports about itself in discovery (same wire fields as the reference)."""

    vendor: str | None
    simulated: bool
    hostname: str
    bridge: str
    probe: Probe
    problems: tuple[str, ...] = ()
    split_test: str = ""
    policy: str = AUTO
    policy_settings: dict[str, Any] = field(default_factory=dict)
    gpu: str | None = None
    pinned_staging: bool = False
    bridge_compression: str = ""
    # B200 additions; absent keys default, so a reference-shaped dictionary still parses.
    islands: tuple[int, ...] = ()
    codec_format: str = "ref"
    fabric: str = "auto"
    pid: int = 0

    @property
    def torch_version(self) -> str:
        return self.probe.torch_version

    def to_wire(self) -> dict[str, Any]:
        return asdict(self)

    @classmethod
    def from_wire(cls, data: dict[str, Any]) -> "PeerInfo":
        data = dict(data)
        probe_data = dict(data.pop("probe"))
        probe_data["errors"] = tuple(probe_data.get("errors", ()))
        data["problems"] = tuple(data.get("problems", ()))
        data["islands"] = tuple(data.get("islands", ()))
        return cls(probe=Probe(**probe_data), **data)


def describe_local(bridge: str, policy: "str | type[CollectivePolicy]" = AUTO
                   ) -> tuple[PeerInfo, Config]:
    """This rank's label, configuration and capabilities.  Whatever would stop it from
    joining becomes an entry of :attr:`PeerInfo.problems` instead of an exception, so that
    discovery fails every rank with one message."""
    import os
    problems: list[str] = []

    def setting(read, default):
        try:
            return read()
        except (ValueError, RuntimeError) as exc:
            problems.append(str(exc))
            return default

    split = setting(_config.split_test_mode, None) or ""
    pinned = setting(_config.pinned_staging_setting, False)
    compression = setting(_config.bridge_compression_setting, "")
    islands = setting(_config.islands_setting, ())
    codec_format = setting(_config.codec_format_setting, "ref")
    fabric = setting(_config.fabric_setting, "auto")
    setting(_config.algo_setting, "auto")
    setting(_config.wait_timeout_ms, 0)
    vendor = setting(detect_vendor, None)
    cfg = setting(_config.resolve_config, None)
    if cfg is None:  # never used to communicate: discovery fails first
        cfg = Config(False, GPU_BACKEND, torch.device("cpu"))
    local_probe = probe()
    if not cfg.simulated and not local_probe.nccl_available:
        problems.append("This PyTorch build has no NCCL backend, so it cannot form a GPU island.")
    settings: dict[str, Any] = {}
    if not isinstance(policy, str):
        try:
            settings = policy.settings()
        except ValueError as exc:
            problems.append(f"Collective policy {policy.name!r}: {exc}")
    info = PeerInfo(
        vendor=vendor, simulated=cfg.simulated, hostname=_config.hostname(cfg.simulated),
        bridge=bridge, probe=local_probe, problems=tuple(problems), split_test=split,
        policy=policy_name(policy), policy_settings=settings, gpu=_config.gpu_identity(cfg.device),
        pinned_staging=pinned, bridge_compression=compression, islands=tuple(islands),
        codec_format=codec_format, fabric=fabric, pid=os.getpid())
    return info, cfg


def _disagree(peers: Sequence[PeerInfo], value, what: str, advice: str) -> None:
    seen: dict[Any, list[int]] = {}
    for rank, peer in enumerate(peers):
        seen.setdefault(value(peer), []).append(rank)
    if len(seen) > 1:
        detail = "; ".join(f"{key!r} on ranks {ranks}" for key, ranks in seen.items())
        raise RuntimeError(f"Ranks {what}: {detail}. {advice}")


def _release_key(release: str):
    return tuple((0, int(p)) if p.isdigit() else (1, p) for p in release.split("."))


def validate_peers(peers: Sequence[PeerInfo], *, warn: bool = True) -> None:
    """Refuse a job in which any rank reported a problem or ranks disagree on how to run
    (reference: topology.py:239-332).  Every rank raises the same text."""
    failing = [(r, p) for r, p in enumerate(peers) if p.problems]
    if failing:
        lines = [f"  rank {r} ({p.hostname}): {problem}" for r, p in failing
                 for problem in p.problems]
        raise RuntimeError(f"gpubridge cannot start: {len(failing)} of {len(peers)} ranks "
                           "reported problems.\n" + "\n".join(lines))
    on_cpu = [r for r, p in enumerate(peers) if p.simulated]
    if on_cpu and len(on_cpu) != len(peers):
        on_gpu = [r for r, p in enumerate(peers) if not p.simulated]
        raise RuntimeError(
            f"Ranks disagree on where to run: ranks {on_cpu} run on CPU ({VENDOR_ENV} or "
            f"{CPU_ONLY_ENV} is set) but ranks {on_gpu} run on GPUs. Use the same mode on "
            "every rank.")
    _disagree(peers, lambda p: p.bridge, "picked different bridge transports",
              "Pass the same bridge on every rank.")
    _disagree(peers, lambda p: p.policy, "picked different collective policies",
              "Pass the same policy on every rank.")
    _disagree(peers, lambda p: json.dumps(p.policy_settings, sort_keys=True),
              f"disagree on the settings of collective policy {peers[0].policy!r}",
              "Set the same GPUBRIDGE_* variables (and thresholds file) on every rank: settings "
              "such as a chunk size decide how many messages a collective sends.")
    _disagree(peers, lambda p: p.split_test or "off", f"disagree on {SPLIT_TEST_ENV}",
              "Set it to the same value on every rank, or on none.")
    _disagree(peers, lambda p: p.pinned_staging, f"disagree on {PINNED_STAGING_ENV}",
              "Set it to the same value on every rank, so a run is one configuration or the other.")
    _disagree(peers, lambda p: p.bridge_compression or "off",
              f"disagree on {BRIDGE_COMPRESSION_ENV}",
              "Set it to the same value on every rank, or on none: it decides what the bridge sends.")
    _disagree(peers, lambda p: tuple(p.islands), f"disagree on {ISLANDS_ENV}",
              "Set it to the same value on every rank, or on none.")
    _disagree(peers, lambda p: p.codec_format, f"disagree on {_config.CODEC_FORMAT_ENV}",
              "Set it to the same value on every rank.")
    _disagree(peers, lambda p: p.fabric, f"disagree on {_config.FABRIC_ENV}",
              "Set it to the same value on every rank.")
    releases = sorted({p.torch_version.split("+")[0] for p in peers}, key=_release_key)
    if warn and len(releases) > 1:
        warnings.warn(f"Ranks run different PyTorch releases ({', '.join(releases)}); prefer "
                      "the same release on every rank.", stacklevel=2)


@dataclass(frozen=True)
class Topology:
    """One rank's view of a group (the world, or a subgroup)."""

    rank: int
    layout: Layout
    peers: tuple[PeerInfo, ...]
    """Every *world* rank's report, indexed by global rank."""
    config: Config
    island_group: Comm
    bridge: BridgeTransport | None
    policy: CollectivePolicy
    transport: type[BridgeTransport] | None = None
    timeout: timedelta | None = None
    world_group: Comm | None = None
    """A Gloo communicator of every member: barrier, flat-gloo, object exchange."""
    cpu_group: Comm | None = None
    """A second Gloo communicator of every member, for CPU tensors handed to the torch
    backend on a GPU job, so its traffic never interleaves with the library's own."""
    fabric: Any = None
    """NVLink symmetric-memory engine of this group, when its members share one box."""
    p2p_group: Comm | None = None
    """GPU jobs: an NCCL communicator of every member that carries send/recv."""
    context: LinkContext | None = None
    """Store and naming scope for links a policy creates in ``setup()``."""

    @property
    def policy_name(self) -> str:
        return self.policy.name

    @property
    def policy_settings(self) -> dict[str, Any]:
        return self.peers[self.rank].policy_settings

    @property
    def pinned_staging(self) -> bool:
        return self.peers[self.rank].pinned_staging

    @property
    def bridge_compression(self) -> str:
        return self.peers[self.rank].bridge_compression

    @property
    def codec_format(self) -> str:
        return self.peers[self.rank].codec_format

    @property
    def bridge_group(self):
        return getattr(self.bridge, "group", None)

    @property
    def world_size(self) -> int:
        return self.layout.world_size

    @property
    def vendor(self) -> str:
        """This rank's island label (differs from :attr:`detected_vendor` when relabelled)."""
        return self.layout.vendors[self.layout.index(self.rank)]

    @property
    def detected_vendor(self) -> str:
        return cast(str, self.peers[self.rank].vendor)

    @property
    def split_test(self) -> str | None:
        me = self.peers[self.rank]
        if me.split_test:
            return me.split_test
        return "islands" if me.islands else None

    @property
    def run_kind(self) -> str:
        if self.split_test:
            return "split-test"
        if self.config.simulated:
            return "cpu"
        return "gpu-mixed" if self.layout.needs_bridge else "gpu-single-vendor"

    @cached_property
    def island(self) -> Island:
        return self.layout.island_of(self.rank)

    @cached_property
    def is_leader(self) -> bool:
        return self.island.leader == self.rank

    @property
    def simulated(self) -> bool:
        return self.config.simulated

    @property
    def device(self) -> torch.device:
        return self.config.device


def gpu_clashes(layout: Layout, hostnames: Sequence[str], gpus: Sequence[str | None]) -> list[str]:
    """Ranks of one island on one GPU (NCCL refuses that), one line per shared GPU.  Islands
    with a rank of unknown GPU (``""``) are skipped; see :func:`unchecked_islands`."""
    lines = []
    for island in layout.islands:
        if any(gpus[r] == "" for r in island.ranks):
            continue
        shared: dict[tuple[str, str], list[int]] = {}
        for r in island.ranks:
            if gpus[r] is not None:
                shared.setdefault((hostnames[r], cast(str, gpus[r])), []).append(r)
        lines += [f"  island {island.vendor!r}: ranks {rs} on {host}, GPU {gpu}"
                  for (host, gpu), rs in shared.items() if len(rs) > 1]
    return lines


def unchecked_islands(layout: Layout, gpus: Sequence[str | None]) -> list[str]:
    return [f"  island {i.vendor!r}: ranks {[r for r in i.ranks if gpus[r] == '']}"
            for i in layout.islands if any(gpus[r] == "" for r in i.ranks)]


def exchange(store, key: str, rank: int, members: Sequence[int], value: Any,
             timeout: timedelta | None = None) -> list[Any]:
    """All-gather of one JSON value per member over the store, in member order."""
    store.set(f"{key}/{rank}", json.dumps(value))
    deadline = time.monotonic() + (timeout or DEFAULT_TIMEOUT).total_seconds()
    keys = [f"{key}/{m}" for m in members]
    while True:
        try:
            store.wait(keys, timedelta(seconds=max(0.05, min(5.0, deadline - time.monotonic()))))
            break
        except Exception:  # noqa: BLE001 - DistStoreError / RuntimeError on timeout
            if time.monotonic() >= deadline:
                missing = [m for m, k in zip(members, keys) if not store.check([k])]
                raise RuntimeError(f"gpubridge discovery: ranks {missing} never reported "
                                   f"({key})") from None
    return [json.loads(store.get(k).decode()) for k in keys]


def labels_for(peers: Sequence[PeerInfo], local: PeerInfo, warn: bool = True) -> list[str]:
    """Island label per world rank: detected vendors, relabelled in a split test."""
    vendors = [cast(str, p.vendor) for p in peers]
    if local.islands:
        labels = island_labels(vendors, local.islands)
        mode = "islands=" + ",".join(map(str, local.islands))
    elif local.split_test:
        labels = split_labels(vendors, [p.hostname for p in peers], local.split_test)
        mode = local.split_test
    else:
        return vendors
    if warn and labels != vendors:
        warnings.warn(banner(mode, vendors, labels), SplitTestWarning, stacklevel=4)
    return labels


def _make_fabric(store, name: str, layout: Layout, rank: int, peers: Sequence[PeerInfo],
                 cfg: Config, timeout: timedelta | None):
    """The NVLink engine for this group, or None (CPU run, switched off, several hosts,
    or the extension is not built)."""
    if cfg.simulated or cfg.device.type != "cuda" or peers[rank].fabric == "off":
        return None
    members = layout.members
    if len({peers[m].hostname for m in members}) != 1:
        return None
    from gpubridge_b200.ops import fabric as _fabric
    return _fabric.create(store, name, layout, rank, cfg.device, timeout)


def build_topology(store, rank: int, world_size: int, local: PeerInfo, cfg: Config, *,
                   transport: type[BridgeTransport],
                   policy: "str | type[CollectivePolicy]" = AUTO,
                   timeout: timedelta | None = None, name: str = "world") -> Topology:
    """Discovery over ``store``, then this rank's communicators, the bridge and the fabric.

    Collective over every rank.  Raises the same ``RuntimeError`` on every rank when a rank
    reported a problem, ranks disagree, two ranks of an island share a GPU, or the policy
    does not fit the layout."""
    members = tuple(range(world_size))
    wire = exchange(store, f"gb/{name}/peer", rank, members, local.to_wire(), timeout)
    peers = tuple(PeerInfo.from_wire(w) for w in wire)
    validate_peers(peers, warn=rank == 0)
    if not cfg.simulated:
        torch.cuda.set_device(cfg.device)   # only now: a bad index failed discovery instead
    labels = labels_for(peers, local)
    layout = plan_topology(labels)
    gpus = [p.gpu for p in peers]
    unchecked = unchecked_islands(layout, gpus)
    if unchecked and rank == 0:
        warnings.warn("gpubridge could not check that ranks of these islands drive different "
                      "GPUs (no UUID or PCI address reported):\n" + "\n".join(unchecked),
                      stacklevel=3)
    clashes = gpu_clashes(layout, [p.hostname for p in peers], gpus)
    if clashes:
        raise RuntimeError(
            "gpubridge cannot start: ranks of one island would share a GPU, and NCCL refuses "
            "two ranks of one communicator on the same GPU.\n" + "\n".join(clashes) +
            "\nStart no more ranks per node than it has GPUs, and check LOCAL_RANK and "
            "CUDA_VISIBLE_DEVICES.")
    return _assemble(store, name, layout, rank, peers, cfg, transport, policy, timeout)


def build_subtopology(world: Topology, store, ranks: Sequence[int], name: str,
                      timeout: timedelta | None = None) -> Topology:
    """A subgroup's own topology over its members only (global ranks, ascending).  Islands
    come from the world's labels; one-label members get ``native-only``, mixed members the
    policy the job asked for and the world's bridge transport over their own leaders
    (reference: topology.py:695-737)."""
    ranks = tuple(ranks)
    labels = [world.layout.vendors[world.layout.index(r)] for r in ranks]
    layout = plan_topology(labels, ranks)
    asked = world.peers[world.rank].policy
    if not layout.needs_bridge or asked == AUTO:
        chosen: "str | type[CollectivePolicy]" = AUTO
    else:
        chosen = type(world.policy)
    assert world.transport is not None
    return _assemble(store, name, layout, world.rank, world.peers, world.config,
                     world.transport, chosen, timeout)


def _assemble(store, name: str, layout: Layout, rank: int, peers, cfg: Config,
              transport: type[BridgeTransport], policy, timeout) -> Topology:
    policy_cls = choose_policy(policy, layout)
    members = layout.members
    world_group = make_comm(store, f"{name}.all", members, rank, "gloo", timeout)
    cpu_group = make_comm(store, f"{name}.cpu", members, rank, "gloo", timeout)
    island = layout.island_of(rank)
    island_group = make_comm(store, f"{name}.island", island.ranks, rank, cfg.island_backend,
                             timeout, cfg.device)
    context = LinkContext(store, rank, name, cfg.device)
    bridge = None
    if layout.needs_bridge:
        bridge = transport.create(layout.bridge_ranks, timeout=timeout, context=context)
        if (bridge is not None) != (rank in layout.bridge_ranks):
            raise RuntimeError(
                f"{transport.__name__}.create() must return a transport exactly on the bridge "
                f"ranks {list(layout.bridge_ranks)}; rank {rank} got {bridge!r}")
    fabric = _make_fabric(store, name, layout, rank, peers, cfg, timeout)
    p2p_group = None
    if not cfg.simulated and cfg.device.type == "cuda":
        p2p_group = make_comm(store, f"{name}.p2p", members, rank, cfg.island_backend, timeout,
                              cfg.device)
    assert island_group is not None and world_group is not None
    topology = Topology(rank=rank, layout=layout, peers=tuple(peers), config=cfg,
                        island_group=island_group, bridge=bridge, policy=policy_cls(),
                        transport=transport, timeout=timeout, world_group=world_group,
                        cpu_group=cpu_group, fabric=fabric, context=context,
                        p2p_group=p2p_group)
    topology.policy.setup(topology)
    _maybe_nvls(topology)
    return topology


def _maybe_nvls(topology: "Topology") -> None:
    """In-switch reduction for the team's SUM / AVG all-reduces of floats.  ``GPUBRIDGE_NVLS``:
    ``1`` (the default) binds switch memory through multicast objects the fabric makes itself -
    the team's and, with several islands, one per island; ``0`` keeps every collective on the
    peer-memory kernels (tests that let a rank leave: a rank that exits while bound to a
    multicast object can fault its peers' links); ``torch`` takes the binding from torch's
    symmetric memory instead (one island, the team must be the whole job)."""
    import os
    fabric = topology.fabric
    setting = os.environ.get("GPUBRIDGE_NVLS", "1").strip().lower()
    if fabric is None or setting in ("0", "off", "false", "no"):
        return
    if setting == "torch":
        import torch.distributed as dist
        if dist.is_initialized() and dist.get_world_size() == topology.world_size:
            fabric.enable_nvls(dist.group.WORLD)
        return
    fabric.enable_switch(timeout=topology.timeout)


def close_topology(topology: Topology) -> None:
    """Release what a topology holds; never raises."""
    for close in (topology.policy.close,
                  getattr(topology.bridge, "close", None),
                  getattr(topology.fabric, "close", None),
                  topology.island_group.close,
                  getattr(topology.world_group, "close", None),
                  getattr(topology.cpu_group, "close", None),
                  getattr(topology.p2p_group, "close", None)):
        if close is None:
            continue
        try:
            close()
        except Exception as exc:  # noqa: BLE001
            warnings.warn(f"gpubridge: closing {close!r} failed: {exc}", RuntimeWarning,
                          stacklevel=2)


_current: Topology | None = None


def get_topology() -> Topology:
    if _current is None:
        raise RuntimeError("gpubridge is not initialized; call gpubridge.init() first")
    return _current


def is_initialized() -> bool:
    return _current is not None


def _set_topology(topology: Topology | None) -> None:
    global _current
    _current = topology
