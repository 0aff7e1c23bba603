"""``dist.init_process_group(backend="gpubridge")``: DDP, FSDP2, HSDP, pipelining and
object collectives through the library.

The method map and the refusals are the reference's (src/gpubridge/torch_backend.py:87-479,
docs/TORCH_BACKEND.md:169-179): ``allreduce(_coalesced)``, ``broadcast``,
``_allgather_base`` / ``all_gather_single``, ``allgather_into_tensor_coalesced``, list
``allgather``, ``_reduce_scatter_base`` / ``reduce_scatter_single``,
``reduce_scatter_tensor_coalesced``, list ``reduce_scatter``, ``barrier``, ``gather`` /
``scatter`` of CPU tensors, coalescing, ``send`` / ``recv``; ``recv_anysource``,
``alltoall*`` and ``reduce`` are refused before any communication.

How it is built differs.  Each group (the world from ``init_process_group``, a subgroup
from ``new_group`` or a ``DeviceMesh`` dimension) gets its own prefix of the job's store
from torch, and the group's topology - discovery, island communicators, bridge, NVLink
fabric - is bootstrapped over that store by the group's members only
(:mod:`gpubridge_b200.groups`).  The world's is built inside ``init_process_group``
itself, which every rank calls; a subgroup's at its first collective.  torch's private
group naming is never patched.

A subgroup whose members share one label is one island (``native-only``: a single fused or
NCCL collective); mixed members get the policy the job asked for.  That is what makes HSDP
work: shard groups are islands, replicate groups cross them (one bridged all_reduce per
gradient shard, compressed if ``GPUBRIDGE_BRIDGE_COMPRESSION`` says so).

On a GPU box every send/recv is an NCCL p2p call (coalesced inside ``batch_isend_irecv``);
in CPU simulation same-island p2p uses the island's Gloo group and cross-island p2p the
host-staged engine of :mod:`gpubridge_b200.p2p`.
"""
from __future__ import annotations

import os
import threading
import time
import warnings
from collections.abc import Callable, Sequence
from datetime import timedelta
from typing import Any

import torch
import torch.distributed as dist
from torch._C._distributed_c10d import _create_work_from_future

from gpubridge_b200 import collectives as _collectives
from gpubridge_b200 import observe as _observe
from gpubridge_b200 import p2p as _p2p
from gpubridge_b200 import topology as _topology
from gpubridge_b200 import work as _work
from gpubridge_b200.config import BRIDGE_ENV, POLICY_ENV, is_simulated
from gpubridge_b200.policies import DEFAULT_POLICY, resolve_policy
from gpubridge_b200.transport import (DEFAULT_TRANSPORT, GlooTransport, NvlinkTransport,
                                      resolve_transport)

NAME = "gpubridge"

_lock = threading.RLock()
_owner: "GpubridgeProcessGroup | None" = None     # the group that owns the world topology
# Jobs of this process so far.  A launcher's store outlives destroy_process_group(), so the
# keys of a second job must not meet the first job's: every name carries the count, which
# all ranks share because every rank creates its world group once per job.
_generation = 0
_subgroups: "list[GpubridgeProcessGroup]" = []


def _completed(result: Any) -> dist.Work:
    future: torch.futures.Future = torch.futures.Future()
    future.set_result(result)
    return _create_work_from_future(future)


def _unsupported(what: str, why: str = "") -> NotImplementedError:
    return NotImplementedError(f"the {NAME} torch.distributed backend doesn't support {what}"
                               + (f": {why}" if why else ""))


class _NoBackend:
    """What ``_get_backend()`` answers: a Python group has no per-device C++ backend."""

    supports_splitting = False
    supports_coalescing = True


def _future_of(work) -> torch.futures.Future:
    try:
        return work.get_future()
    except RuntimeError as exc:
        if "not implemented" not in str(exc):
            raise
    work.wait()
    future: torch.futures.Future = torch.futures.Future()
    future.set_result(None)
    return future


def _all_of(works: Sequence, result: Any) -> dist.Work:
    futures = [_future_of(w) for w in works]
    if not futures:
        return _completed(result)
    return _create_work_from_future(torch.futures.collect_all(futures).then(
        lambda f: ([g.value() for g in f.value()], result)[1]))


class _BatchWork(dist.Work):
    """The Work of a coalesced batch: waits on each member itself, so a slow future
    callback elsewhere never delays it and a finite timeout works."""

    def __init__(self, works: Sequence, future: torch.futures.Future) -> None:
        super().__init__()
        self._works, self._future = list(works), future

    def wait(self, timeout: timedelta | None = None) -> bool:
        end = None if timeout is None else time.monotonic() + timeout.total_seconds()
        for work in self._works:
            if end is None:
                work.wait()
            else:
                work.wait(timedelta(seconds=max(0.0, end - time.monotonic())))
        return True

    def is_completed(self) -> bool:
        return all(w.is_completed() for w in self._works)

    def is_success(self) -> bool:
        return self.is_completed() and self.exception() is None

    def exception(self):
        for w in self._works:
            error = w.exception()
            if error is not None:
                return error
        return None

    def get_future(self):
        return self._future

    def synchronize(self) -> None:
        self.wait()


class GpubridgeProcessGroup(dist.ProcessGroup):
    """The world group, or a subgroup with ``members`` (its global ranks, ascending)."""

    def __init__(self, rank: int, size: int, name: str, timeout: timedelta | None,
                 members: Sequence[int] = (), store=None) -> None:
        super().__init__(rank, size)
        self._name, self._timeout = name, timeout
        self._members = tuple(members)
        self._store = store
        self._built: _topology.Topology | None = None
        self._build_lock = threading.Lock()
        self._building = False
        self._coalesced: list | None = None
        self._coalesced_torch: list = []
        self._native_batch = None
        self._engine: _p2p.Engine | None = None
        self._engine_lock = threading.Lock()
        global _generation
        if not self._members:
            _generation += 1
        self._generation = _generation
        self._p2p_store = (dist.PrefixStore(f"gpubridge-p2p{self._generation}", store)
                           if store is not None else None)
        self._on_shutdown: Callable[[], None] | None = None     # set by the C++ front end's glue

    # -- identity ----------------------------------------------------------------------------
    @property
    def group_name(self) -> str:
        return self._name

    @property
    def pg_name(self) -> str:
        return self._name

    def getBackendName(self) -> str:  # noqa: N802 - torch's name
        return NAME

    def _get_backend(self, device):
        return _NoBackend()

    def __repr__(self) -> str:
        extra = f", members={list(self._members)}" if self._members else ""
        return f"GpubridgeProcessGroup(rank={self.rank()}, size={self.size()}{extra})"

    def _global(self, group_rank: int) -> int:
        return self._members[group_rank] if self._members else group_rank

    # -- topology ----------------------------------------------------------------------------
    def _build_world(self) -> None:
        """Discovery and the world's communicators, over this group's store."""
        global _owner
        with _lock:
            if _owner is not None:
                return
            if _topology.is_initialized():
                raise RuntimeError("gpubridge is already initialized in this process "
                                   f"(gpubridge.init()); use either init() or the {NAME} backend")
            problems: list[str] = []
            transport, chosen = GlooTransport, DEFAULT_POLICY
            try:
                default = DEFAULT_TRANSPORT if is_simulated() else NvlinkTransport.name
                transport = resolve_transport(os.environ.get(BRIDGE_ENV, "").strip() or default)
                chosen = resolve_policy(os.environ.get(POLICY_ENV, "").strip() or DEFAULT_POLICY)
            except (ValueError, TypeError) as exc:
                problems.append(str(exc))
            try:
                local, cfg = _topology.describe_local(transport.name, chosen)
            except (ValueError, TypeError) as exc:       # e.g. a bad GPUBRIDGE_VENDOR
                problems.append(str(exc))
                from gpubridge_b200.config import Config
                from gpubridge_b200.detect import probe
                cfg = Config(True, "gloo", torch.device("cpu"))
                local = _topology.PeerInfo(None, True, "?", transport.name, probe())
            if problems:
                local = _topology.PeerInfo(**{**local.__dict__,
                                              "problems": (*local.problems, *problems)})
            topology = _topology.build_topology(
                self._store, self.rank(), self.size(), local, cfg, transport=transport,
                policy=chosen, timeout=self._timeout, name=f"pg{self._generation}")
            _work.shutdown()
            _observe._reset()
            _topology._set_topology(topology)
            _owner = self

    def _topology(self) -> _topology.Topology:
        self._check_p2p()
        default = _default_group(self)
        default._build_world()
        world = _topology.get_topology()
        if not self._members:
            return world
        with self._build_lock:
            if self._built is None:
                if self._building:
                    raise RuntimeError(f"a collective on a {NAME} subgroup ran while that "
                                       "subgroup was setting itself up")
                self._building = True
                try:
                    self._built = _topology.build_subtopology(world, self._store, self._members,
                                                              f"sub{self._generation}", self._timeout)
                finally:
                    self._building = False
                with _lock:
                    _subgroups.append(self)
            return self._built

    def _cpu(self):
        return self._topology().cpu_group

    # -- the C++ front end (native_backend.py) asks these ------------------------------------------
    def _native_team(self):
        """``(engine, stream, device index, grid cap, team rank of each group rank)`` when this
        group's collectives on CUDA tensors can be planned and launched by the native engine,
        else None: no NVLink fabric, a compressed bridge, or a policy that shapes the fused
        kernel differently (pipelined, sharded, auto-tuned)."""
        from gpubridge_b200 import policies as _policies
        topology = self._topology()
        fabric, policy = topology.fabric, topology.policy
        if fabric is None or type(policy) not in (_policies.ReduceBridgeBroadcast, _policies.NativeOnly):
            return None
        if getattr(policy, "_mode", ""):
            return None
        engine = fabric.engine()
        if not engine:
            return None
        team_rank = [fabric.layout.index(self._global(r)) for r in range(self.size())]
        return (engine, fabric.comm_stream.cuda_stream, fabric.device.index, fabric.overlap_blocks,
                team_rank)

    def _native_failed(self) -> None:
        """A device-side wait of this team ran out: raise what the kernel recorded."""
        self._topology().fabric.check()

    def shutdown(self) -> None:
        """Called by ``destroy_process_group()``; releases state without running what is
        queued and never raises."""
        if self._engine is not None:
            self._engine.close()
        released, self._on_shutdown = self._on_shutdown, None
        if released is not None:
            released()
        if self._members:
            _close_subgroup(self)
        else:
            _teardown(self)

    def abort(self) -> None:
        self.shutdown()

    # -- running collectives -------------------------------------------------------------------
    def _run(self, what: str, result: Any, calls: Sequence[Callable[[], "_work.Work | None"]]
             ) -> dist.Work:
        works: list[_work.Work] = []
        try:
            for call in calls:
                work = call()
                assert work is not None
                works.append(work)
        except (ValueError, TypeError, NotImplementedError) as exc:
            raise type(exc)(f"{NAME} backend, {what}: {exc}") from exc
        if self._coalesced is not None:
            self._coalesced.extend(works)
        if not works:
            return _completed(result)

        def done(future: torch.futures.Future) -> Any:
            future.value()
            for work in works[:-1]:
                if work.exception() is not None:
                    raise RuntimeError(f"{NAME} backend, {what} failed") from work.exception()
            return result

        return _create_work_from_future(works[-1].get_future().then(done))

    def _on_cpu(self, result: Any, starts: Sequence[Callable[[], Any]]) -> dist.Work:
        works = [w for w in (start() for start in starts) if w is not None]
        if self._coalesced is not None:
            self._coalesced_torch.extend(works)
        return _all_of(works, result)

    # -- collectives -----------------------------------------------------------------------------
    def allreduce(self, tensors, opts=None):  # noqa: D102
        op = opts.reduceOp if opts is not None else dist.ReduceOp.SUM
        topology = self._topology()
        if _cpu_path(topology, tensors):
            name = _check_op(op, "allreduce")
            return self._on_cpu(list(tensors), [
                lambda t=t: _gloo_reduce(self._cpu(), t, name, self.size()) for t in tensors])
        return self._run("allreduce", list(tensors), [
            lambda t=t: _collectives.all_reduce(t, op=op, async_op=True, _topology=topology)
            for t in tensors])

    def allreduce_coalesced(self, tensors, opts=None):  # noqa: D102
        return self.allreduce(tensors, opts)

    def broadcast(self, tensors, opts=None):  # noqa: D102
        root = self._global(opts.rootRank if opts is not None else 0)
        topology = self._topology()
        if _cpu_path(topology, tensors):
            return self._on_cpu(list(tensors), [
                lambda t=t: self._cpu().broadcast(t, root, async_op=True) for t in tensors])
        return self._run("broadcast", list(tensors), [
            lambda t=t: _collectives.broadcast(t, root, async_op=True, _topology=topology)
            for t in tensors])

    def _allgather_base(self, output, input, opts=None):  # noqa: A002, D102
        return self.allgather_into_tensor_coalesced([output], [input], opts)

    all_gather_single = _allgather_base

    def allgather_into_tensor_coalesced(self, outputs, inputs, opts=None):  # noqa: D102
        topology = self._topology()
        if _cpu_path(topology, [*outputs, *inputs]):
            return self._on_cpu(list(outputs), [
                lambda o=o, i=i: _gloo_all_gather(self._cpu(), o, i)
                for o, i in zip(outputs, inputs)])
        return self._run("all_gather_into_tensor", list(outputs), [
            lambda o=o, i=i: _collectives.all_gather_into_tensor(
                _flat(o), _flat(i), async_op=True, _topology=topology)
            for o, i in zip(outputs, inputs)])

    all_gather_single_coalesced = allgather_into_tensor_coalesced

    def allgather(self, output_lists, inputs, opts=None):  # noqa: D102
        """List form (DDP's parameter-shape check): one gather per input, copied out."""
        topology = self._topology()
        for outputs, tensor in zip(output_lists, inputs):
            if len(outputs) != self.size() or any(o.shape != tensor.shape for o in outputs):
                raise _unsupported("allgather with tensors of different sizes",
                                   "every rank must contribute a tensor of the same shape")
        on_cpu = _cpu_path(topology, inputs)
        for outputs, tensor in zip(output_lists, inputs):
            buffer = torch.empty(self.size() * tensor.numel(), dtype=tensor.dtype,
                                 device=tensor.device)
            source = tensor.contiguous().reshape(-1)
            if on_cpu:
                self._cpu().all_gather_into(buffer, source)
            else:
                # a blocking call of a fused collective is ordered on the current stream, so
                # the copies below see the gathered rows (a Work whose result holds no tensor
                # would carry no device events to wait on)
                try:
                    _collectives.all_gather_into_tensor(buffer, source, _topology=topology)
                except (ValueError, TypeError, NotImplementedError) as exc:
                    raise type(exc)(f"{NAME} backend, allgather: {exc}") from exc
            for out, row in zip(outputs, buffer.view(self.size(), *tensor.shape).unbind(0)):
                out.copy_(row)
        return _completed(output_lists)

    def _reduce_scatter_base(self, output, input, opts=None):  # noqa: A002, D102
        return self.reduce_scatter_tensor_coalesced([output], [input], opts)

    reduce_scatter_single = _reduce_scatter_base

    def reduce_scatter_tensor_coalesced(self, outputs, inputs, opts=None):  # noqa: D102
        op = opts.reduceOp if opts is not None else dist.ReduceOp.SUM
        topology = self._topology()
        if _cpu_path(topology, [*outputs, *inputs]):
            name = _check_op(op, "reduce_scatter_tensor")
            if name not in ("sum", "avg"):
                raise _unsupported(f"reduce_scatter with {name.upper()}", "SUM and AVG only")
            return self._on_cpu(list(outputs), [
                lambda o=o, i=i: _gloo_reduce_scatter(self._cpu(), o, i, name, self.size())
                for o, i in zip(outputs, inputs)])
        return self._run("reduce_scatter_tensor", list(outputs), [
            lambda o=o, i=i: _collectives.reduce_scatter_tensor(
                _flat(o), _flat(i), op=op, async_op=True, _topology=topology)
            for o, i in zip(outputs, inputs)])

    reduce_scatter_single_coalesced = reduce_scatter_tensor_coalesced

    def reduce_scatter(self, outputs, input_lists, opts=None):  # noqa: D102
        joined = []
        for output, slices in zip(outputs, input_lists):
            if len(slices) != self.size() or any(s.shape != output.shape for s in slices):
                raise _unsupported("reduce_scatter with slices of different sizes",
                                   "every slice must have the output's shape")
            joined.append(torch.cat([s.reshape(-1) for s in slices]))
        return self.reduce_scatter_tensor_coalesced(list(outputs), joined, opts)

    # the names later torch releases give the same entry points (reference:
    # docs/TORCH_BACKEND.md:169-179)
    def all_gather_single(self, output, input, opts=None):  # noqa: A002, D102
        return self._allgather_base(output, input, opts)

    def all_gather_single_coalesced(self, outputs, inputs, opts=None):  # noqa: D102
        return self.allgather_into_tensor_coalesced(outputs, inputs, opts)

    def reduce_scatter_single(self, output, input, opts=None):  # noqa: A002, D102
        return self._reduce_scatter_base(output, input, opts)

    def barrier(self, opts=None):  # noqa: D102
        topology = self._topology()
        return self._run("barrier", [], [
            lambda: _collectives.barrier(async_op=True, _topology=topology)])

    def gather(self, outputs, inputs, opts=None):  # noqa: D102
        """CPU tensors only (what ``gather_object`` and checkpoint planning need)."""
        root = opts.rootRank if opts is not None else 0
        _cpu_only("gather", [*inputs, *(t for lst in outputs for t in lst)])
        comm = self._cpu()
        rows = outputs[0] if self.rank() == root else None
        comm.gather(inputs[0], rows, self._global(root))
        return _completed(outputs)

    def scatter(self, outputs, inputs, opts=None):  # noqa: D102
        root = opts.rootRank if opts is not None else 0
        _cpu_only("scatter", [*outputs, *(t for lst in inputs for t in lst)])
        comm = self._cpu()
        slices = inputs[0] if self.rank() == root else None
        comm.scatter(outputs[0], slices, self._global(root))
        return _completed(outputs)

    # -- coalescing ------------------------------------------------------------------------------
    def _start_coalescing(self, device) -> None:
        self._coalesced, self._coalesced_torch = [], []

    def _end_coalescing(self, device) -> dist.Work:
        if self._native_batch is not None:
            native, self._native_batch = self._native_batch, None
            self._coalesced_torch.append(native._end_coalescing())
        works, self._coalesced = self._coalesced or [], None
        torch_works, self._coalesced_torch = self._coalesced_torch, []
        futures, members = [], list(works)
        for work in torch_works:
            try:
                futures.append(work.get_future())
                members.append(work)
            except RuntimeError as exc:
                if "not implemented" not in str(exc):
                    raise
                futures.append(_future_of(work))    # Gloo p2p: wait now, once
        if works:
            futures.append(works[-1].get_future())
        if not futures:
            return _completed([])
        return _BatchWork(members, torch.futures.collect_all(futures).then(
            lambda f: ([g.value() for g in f.value()], [])[1]))

    # -- point-to-point --------------------------------------------------------------------------
    def _check_p2p(self) -> None:
        if self._engine is not None:
            self._engine.check()
        elif self._p2p_store is not None and self._p2p_store.check(["failure"]):
            raise RuntimeError(self._p2p_store.get("failure").decode())

    def _point_to_point(self, tensors, peer: int, tag: int, sending: bool):
        if len(tensors) != 1:
            raise ValueError("gpubridge point-to-point takes exactly one tensor")
        tensor = tensors[0]
        if tensor.layout != torch.strided or not tensor.is_contiguous():
            raise ValueError("gpubridge point-to-point takes contiguous dense tensors")
        if not 0 <= peer < self.size():
            raise ValueError(f"point-to-point peer {peer} is outside this group")
        if not isinstance(tag, int) or not 0 <= tag < 2**31:
            raise ValueError("point-to-point tag must be an integer in [0, 2**31)")
        # Setup is collective; P2P may involve two members only.  Refuse locally rather than
        # rendezvous with ranks that never entered this call.
        if _owner is None or (self._members and self._built is None):
            raise RuntimeError("gpubridge point-to-point needs topology setup first; call "
                               "dist.barrier() on this group first")
        topology = self._topology()
        if tensor.device.type != "cpu" and tensor.device != topology.device:
            raise ValueError(f"point-to-point tensor is on {tensor.device}, expected "
                             f"{topology.device} or cpu")
        target = self._global(peer)
        cuda = tensor.device.type == "cuda"
        comm = None
        if cuda and topology.p2p_group is not None:
            comm = topology.p2p_group               # NCCL p2p, any island
        elif target in topology.island.ranks:
            comm = (topology.cpu_group if tensor.device.type == "cpu"
                    and topology.device.type != "cpu" else topology.island_group)
        if comm is not None:
            batch = self._coalesced is not None and cuda
            if batch and self._native_batch is None:
                comm.backend._start_coalescing()
                self._native_batch = comm.backend
            work = (comm.send if sending else comm.recv)(tensor, target, tag)
            if self._coalesced is not None and not batch:
                self._coalesced_torch.append(work)
            return work
        with self._engine_lock:
            if self._engine is None:
                link = topology.transport.create_p2p(topology.world_group,
                                                     store=self._p2p_store, timeout=self._timeout)
                self._engine = _p2p.Engine(link, topology.device, topology.rank, self._p2p_store,
                                           self._timeout, pinned=topology.pinned_staging,
                                           chunk_bytes=_p2p.chunk_bytes_setting())
        work = self._engine.submit(tensor, target, tag, sending)
        wrapped = _p2p.TorchWork(work, peer if not sending else self.rank())
        if self._coalesced is not None:
            self._coalesced_torch.append(wrapped)
        return wrapped

    def send(self, tensors, dst: int, tag: int):  # noqa: D102
        return self._point_to_point(tensors, dst, tag, True)

    def recv(self, tensors, src: int, tag: int):  # noqa: D102
        return self._point_to_point(tensors, src, tag, False)

    # -- refused -----------------------------------------------------------------------------------
    def recv_anysource(self, *a, **k):  # noqa: D102
        raise _unsupported("any-source recv", "specify src so the route is known")

    def alltoall(self, *a, **k):  # noqa: D102
        raise _unsupported("all_to_all")

    def alltoall_base(self, *a, **k):  # noqa: D102
        raise _unsupported("all_to_all_single")

    def all_to_all_single(self, *a, **k):  # noqa: D102
        raise _unsupported("all_to_all_single")

    def reduce(self, *a, **k):  # noqa: D102
        raise _unsupported("reduce", "use all_reduce")


def _flat(tensor: torch.Tensor) -> torch.Tensor:
    return tensor if tensor.dim() == 1 or not tensor.is_contiguous() else tensor.view(-1)


def _cpu_path(topology, tensors) -> bool:
    """CPU tensors on a GPU job: the group's second Gloo communicator carries them."""
    return topology.device.type != "cpu" and all(t.device.type == "cpu" for t in tensors)


def _cpu_only(what: str, tensors) -> None:
    if not all(t.device.type == "cpu" for t in tensors):
        raise _unsupported(f"{what} of GPU tensors",
                           f"{what} runs on Gloo, for CPU tensors (e.g. {what}_object)")


def _check_op(op, what: str) -> str:
    try:
        return _collectives._op_name(op, what)
    except ValueError as exc:
        raise ValueError(f"{NAME} backend, {what}: {exc}") from exc


def _gloo_reduce(comm, tensor, name: str, size: int):
    comm.all_reduce(tensor, "sum" if name == "avg" else name)
    if name == "avg":
        tensor.div_(size)
    return None


def _gloo_all_gather(comm, output, input):  # noqa: A002
    if output.is_contiguous():
        comm.all_gather_into(output.view(-1), input.reshape(-1))
    else:
        flat = output.new_empty(output.numel())
        comm.all_gather_into(flat, input.reshape(-1))
        output.copy_(flat.view(output.shape))
    return None


def _gloo_reduce_scatter(comm, output, input, name: str, size: int):  # noqa: A002
    flat = output.view(-1) if output.is_contiguous() else output.new_empty(output.numel())
    comm.reduce_scatter_into(flat, input.reshape(-1))
    if name == "avg":
        flat.div_(size)
    if flat.data_ptr() != output.data_ptr():
        output.copy_(flat.view(output.shape))
    return None


def _default_group(group: GpubridgeProcessGroup) -> GpubridgeProcessGroup:
    if _owner is not None:
        return _owner
    try:
        default = dist.distributed_c10d._get_default_group()
    except (RuntimeError, ValueError):
        return group
    return default if isinstance(default, GpubridgeProcessGroup) else group


def _close_subgroup(group: GpubridgeProcessGroup) -> None:
    with _lock:
        if group in _subgroups:
            _subgroups.remove(group)
        built, group._built = group._built, None
    if built is not None:
        _topology.close_topology(built)


def _teardown(group: GpubridgeProcessGroup) -> None:
    global _owner
    with _lock:
        if _owner is not group:
            return
        _owner = None
        subs = list(_subgroups)
        if not _topology.is_initialized():
            return
        try:
            from gpubridge_b200 import _release
            _release(drain=False)
        except Exception as exc:  # noqa: BLE001 - destroy_process_group must finish
            warnings.warn(f"{NAME} backend: releasing gpubridge's state failed: {exc}",
                          RuntimeWarning, stacklevel=3)
    for sub in subs:
        _close_subgroup(sub)


def front_end() -> str:
    """Which object answers ``backend="gpubridge"``: ``native`` - the C++ ``c10d::Backend`` of
    :mod:`gpubridge_b200.native_backend`, with the Python group behind it for everything off
    the hot path - or ``python``.  ``GPUBRIDGE_FRONT_END`` decides; unset (``auto``) it is the
    C++ front end on GPU ranks and the Python group in CPU simulation."""
    setting = os.environ.get("GPUBRIDGE_FRONT_END", "auto").strip().lower() or "auto"
    if setting not in ("auto", "native", "python"):
        raise ValueError(f"GPUBRIDGE_FRONT_END={setting!r}: expected auto, native or python")
    if setting != "auto":
        return setting
    from gpubridge_b200.config import is_simulated
    import torch
    if os.environ.get("GPUBRIDGE_BOUNDS", "0") == "1":
        return "python"         # the C++ front end is linked against the unchecked library
    return "native" if torch.cuda.is_available() and not is_simulated() else "python"


def create(options, backend_options=None):
    """The creator torch calls (``extended_api=True``) on a group's members: the C++ front end
    or the Python process group, as :func:`front_end` says.  If the C++ module cannot be
    loaded on an ``auto`` choice the Python group answers, with a warning."""
    choice = front_end()
    if choice == "native":
        from gpubridge_b200 import native_backend
        try:
            return native_backend.create(options, backend_options)
        except (ImportError, OSError, RuntimeError) as failure:
            if os.environ.get("GPUBRIDGE_FRONT_END", "auto").strip().lower() == "native":
                raise
            import warnings
            warnings.warn(f"gpubridge: the C++ front end could not be loaded ({failure}); "
                          "using the Python process group", RuntimeWarning, stacklevel=2)
    return create_python(options, backend_options)


def create_python(options, backend_options=None) -> GpubridgeProcessGroup:
    """The Python process group of a new group.  The world's topology is built here, inside
    ``init_process_group``, which every rank calls."""
    ranks = list(options.global_ranks_in_group)
    if ranks != sorted(ranks):
        raise RuntimeError(f"the {NAME} torch.distributed backend takes a subgroup's ranks in "
                           f"ascending order, but got {ranks}: new_group(..., sort_ranks=False) "
                           "isn't supported")
    world = dist.get_world_size() if dist.is_initialized() else options.group_size
    members = ranks if ranks and ranks != list(range(world)) else []
    group = GpubridgeProcessGroup(options.group_rank, options.group_size, options.group_id,
                                  options.timeout, members, options.store)
    if not members and _owner is None and not dist.is_initialized():
        group._build_world()
    return group


def register() -> None:
    """Make ``backend="gpubridge"`` known to ``torch.distributed`` (idempotent)."""
    if dist.is_available() and NAME not in dist.Backend.backend_list:
        dist.Backend.register_backend(NAME, create, extended_api=True, devices=["cpu", "cuda"])


def batch_isend_irecv(operations):
    """A coalesced P2P batch: torch's own helper leaves Python process groups out of its
    coalescing path, so native GPU ops of one batch would not be grouped."""
    dist.distributed_c10d._check_p2p_op_list(operations)
    group = operations[0].group or dist.distributed_c10d._get_default_group()
    if not isinstance(group, GpubridgeProcessGroup):
        return dist.batch_isend_irecv(operations)
    device = operations[0].tensor.device
    with dist.distributed_c10d._coalescing_manager(group, device, async_ops=True) as cm:
        for op in operations:
            op.op(op.tensor, group=op.group, tag=op.tag,
                  **{"group_dst" if op.op is dist.isend else "group_src": op.group_peer})
    return cm.works
