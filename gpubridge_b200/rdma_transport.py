"""The bridge transport over the RDMA-style endpoint: where a message's bytes are taken from.

An adapter reads and writes *registered* memory.  For every tensor the bridge carries, a
:class:`Router` picks one of three ways to give the endpoint registered bytes:

``in-place``  the tensor's own device memory is registered and the adapter works on it
              directly (GPUDirect RDMA); needs a provider that registers device memory and a
              device whose direct writes can be made visible (:mod:`gpubridge_b200.gdr`);
``plain``     a contiguous host tensor is handed over as it lies; the endpoint's registration
              cache keeps its registration for the next call on the same buffer;
``bounce``    everything else (device tensors without a direct path, small device tensors
              where a registration costs more than a copy, non-contiguous tensors) goes
              through a :class:`RegisteredStaging` buffer: pinned host memory whose
              registration stays cached, copied in pieces so that the device copy of piece
              ``i + 1`` overlaps the network's work on piece ``i``.

:class:`RdmaTransport` is the ``verbs`` bridge: a :class:`~gpubridge_b200.tagged.TaggedBridge`
whose worker is an :class:`~gpubridge_b200.rdma.Endpoint`.  Across machines it needs a provider
over real queue pairs, which this build does not have (``rdma.load`` says so on every rank);
``RdmaTransport.over_fabric`` builds it over the in-process fabric, which is how the routing,
the staging and the failure rule are tested (reference: verbs/transport.py - Router,
RegisteredStaging, staged chunk overlap).
"""
from __future__ import annotations

import collections
import dataclasses
import time
from datetime import timedelta
from typing import Sequence

import torch

from gpubridge_b200 import config as _config
from gpubridge_b200 import gdr as _gdr
from gpubridge_b200 import rdma as _rdma
from gpubridge_b200.tagged import DTYPE_CODES, OP_CODES, OnDevice, TaggedBridge

#: endpoint settings of ``bridge="verbs"``: variable -> (endpoint argument, default, must be a multiple of)
ENDPOINT_SETTINGS = {
    "GPUBRIDGE_VERBS_SLOT_BYTES": ("eager_max", 16 << 10, 8),          # largest message that travels in a receive slot
    "GPUBRIDGE_VERBS_CREDITS": ("data_slots", 16, 1),                  # receive slots (= send credits) per peer
    "GPUBRIDGE_VERBS_WRITE_BYTES": ("max_write", 1 << 20, 8),          # size of one remote write of a large message
    "GPUBRIDGE_VERBS_UNEXPECTED_BYTES": ("unexpected_max", 64 << 20, 1),   # early messages kept per endpoint
    "GPUBRIDGE_VERBS_MR_CACHE": ("mr_cache", 64, 1),                   # registrations kept, least recently used out
}
GPU_PATH_ENV = "GPUBRIDGE_VERBS_GPU_PATH"          # auto | staged: staged keeps device tensors off the direct path
OBSERVE_ENV = "GPUBRIDGE_VERBS_OBSERVE"            # a file: one JSON line per bridge call, the counters at close
OBSERVE_QUEUE_ENV = "GPUBRIDGE_VERBS_OBSERVE_QUEUE"
JOB_ENV = "GPUBRIDGE_JOB_ID"
DIRECT_MIN_ENV = "GPUBRIDGE_VERBS_DIRECT_MIN_BYTES"
STAGING_ENV = "GPUBRIDGE_VERBS_STAGING_BYTES"
PIECE_ENV = "GPUBRIDGE_VERBS_PIECE_BYTES"


@dataclasses.dataclass(frozen=True)
class Route:
    how: str            # "in-place", "plain" or "bounce"
    why: str


class Router:
    """Decides, per tensor, where the endpoint takes the bytes from.  Pure: the same inputs
    give the same route on every member, so both ends of a link agree without talking."""

    def __init__(self, *, device_registration: bool = False, direct_min_bytes: int | None = None,
                 flush_plans=None, registrar=None) -> None:
        self.device_registration = device_registration or registrar is not None
        #: a :class:`gpubridge_b200.rdma_direct.Registrar`: asked whether THIS range can be
        #: registered (dma-buf or peer memory); its reasons become the route's when it cannot
        self.registrar = registrar
        self.direct_min = (_config.size_setting(DIRECT_MIN_ENV, 64 << 10, multiple=1)
                           if direct_min_bytes is None else direct_min_bytes)
        self._plans = flush_plans or _gdr.plan
        self.gpu_path = _config.choice(GPU_PATH_ENV, ("auto", "staged"), "auto")
        self.counts = collections.Counter()

    def plan(self, device: int):
        """The flush plan of ``device`` this router decides by."""
        return self._plans(device)

    def route(self, tensor: torch.Tensor) -> Route:
        chosen = self._route(tensor)
        self.counts[chosen.how] += 1
        return chosen

    def _route(self, tensor: torch.Tensor) -> Route:
        if not tensor.is_contiguous():
            return Route("bounce", "the tensor is not contiguous")
        if tensor.device.type == "cpu":
            return Route("plain", "contiguous host memory is registered where it lies")
        if self.gpu_path == "staged":
            return Route("bounce", f"{GPU_PATH_ENV}=staged keeps device tensors off the direct path")
        if not self.device_registration:
            return Route("bounce", "the provider cannot register device memory")
        if tensor.nbytes < self.direct_min:
            return Route("bounce", f"below {self.direct_min} bytes a copy is cheaper than a registration")
        plan = self._plans(tensor.device.index or 0)
        if not plan.direct_ok:
            return Route("bounce", plan.reason)
        if self.registrar is not None:
            from gpubridge_b200.rdma_direct import NotDirect
            try:
                region = self.registrar.take(tensor.data_ptr(), tensor.nbytes)
            except NotDirect as reasons:
                return Route("bounce", f"the range cannot be registered ({reasons})")
            self.registrar.give_back(region)               # stays cached for the call that follows
            return Route("in-place", f"registered through {region.method}; {plan.reason}")
        return Route("in-place", plan.reason)


class RegisteredStaging:
    """Pinned host buffers the endpoint keeps registered: one per power-of-two size class,
    least recently used first out when the budget is exceeded (its registrations are dropped
    from the endpoint's cache before the memory goes)."""

    def __init__(self, endpoint, budget_bytes: int | None = None, pin: bool | None = None) -> None:
        self.endpoint = endpoint
        self.budget = (_config.size_setting(STAGING_ENV, 256 << 20, multiple=1)
                       if budget_bytes is None else budget_bytes)
        self.pin = torch.cuda.is_available() if pin is None else pin
        self._buffers: "collections.OrderedDict[int, torch.Tensor]" = collections.OrderedDict()
        self.allocated = self.reused = self.evicted = 0

    def held_bytes(self) -> int:
        return sum(b.numel() for b in self._buffers.values())

    def take(self, nbytes: int) -> torch.Tensor:
        """A byte buffer of at least ``nbytes``; the same size class gives the same buffer."""
        size = 1 << max(12, (max(1, nbytes) - 1).bit_length())
        buffer = self._buffers.pop(size, None)
        if buffer is None:
            while self._buffers and self.held_bytes() + size > self.budget:
                _, victim = self._buffers.popitem(last=False)
                self.endpoint.invalidate(victim.data_ptr(), victim.numel())
                self.evicted += 1
            buffer = torch.empty(size, dtype=torch.uint8, pin_memory=self.pin)
            self.allocated += 1
        else:
            self.reused += 1
        self._buffers[size] = buffer          # most recently used last
        return buffer

    def close(self) -> None:
        for buffer in self._buffers.values():
            self.endpoint.invalidate(buffer.data_ptr(), buffer.numel())
        self._buffers.clear()


def endpoint_settings() -> dict[str, int]:
    """The endpoint arguments the ``GPUBRIDGE_VERBS_*`` variables ask for (defaults where unset)."""
    return {argument: _config.size_setting(name, default, multiple=multiple)
            for name, (argument, default, multiple) in ENDPOINT_SETTINGS.items()}


_emitters: dict[str, object] = {}


def observations(rank: int | None = None):
    """The process's emitter of bridge observations (``GPUBRIDGE_VERBS_OBSERVE=FILE``; ``%r`` in the
    name becomes the rank, so that ranks do not share a file), or None.  One JSON line per bridge
    call - bridge, member, bytes, route, milliseconds or the failure - and the endpoint's counters
    when a bridge closes; written behind a bounded queue (``GPUBRIDGE_VERBS_OBSERVE_QUEUE``
    records) by :class:`gpubridge_b200.telemetry.Emitter`, labelled with ``GPUBRIDGE_JOB_ID``."""
    import atexit
    import os
    path = os.environ.get(OBSERVE_ENV, "").strip()
    if not path:
        return None
    path = path.replace("%r", str(rank) if rank is not None else os.environ.get("RANK", "0"))
    if path not in _emitters:
        from gpubridge_b200.telemetry import Emitter
        capacity = _config.size_setting(OBSERVE_QUEUE_ENV, 4096, multiple=1)
        made = Emitter(path, capacity=capacity, job=os.environ.get(JOB_ENV, "").strip() or None, pid=os.getpid())
        atexit.register(made.close)
        _emitters[path] = made
    return _emitters[path]


class RdmaTransport(TaggedBridge):
    """Registered under its name by ``rdma.load`` once a provider over real queue pairs is
    part of the build; until then resolving ``bridge="verbs"`` says why it cannot load."""

    name = "verbs"
    device_tensors = True
    _instead = 'use bridge="multitcp" or bridge="gloo" across machines'

    def __init__(self, worker, members: Sequence[int], rank: int, timeout: timedelta,
                 chunk_bytes: int, router: Router | None = None,
                 staging: RegisteredStaging | None = None, piece_bytes: int | None = None) -> None:
        super().__init__(worker, members, rank, timeout, chunk_bytes)
        self.router = router or Router()
        self.staging = staging or RegisteredStaging(worker)
        self.piece_bytes = (_config.size_setting(PIECE_ENV, 8 << 20, multiple=256)
                            if piece_bytes is None else piece_bytes)
        self._copy_stream = None
        self.last_route: Route | None = None
        self.observations = observations(rank)

    @classmethod
    def _connect(cls, store, key, members, rank, timeout, deadline):
        if not _rdma.provider_available():
            _rdma.load(cls.name)               # raises: no provider over real queue pairs here
        # the socket provider: every member publishes its socket name on the store
        from gpubridge_b200.tagged import wait_for_keys
        index = list(members).index(rank)
        tcp_host = None
        if _rdma.provider_kind() == "tcp":
            from gpubridge_b200.multitcp import listen_address
            tcp_host = listen_address()
        settings = endpoint_settings()              # a bad value fails here, on this leader
        chunk = _config.size_setting("GPUBRIDGE_VERBS_CHUNK_BYTES", 4 << 20)
        # both ends of a link must cut messages alike and offer the slots the other end counts on
        import json
        store.set(f"{key}/settings/{rank}", json.dumps(dict(settings, chunk_bytes=chunk), sort_keys=True))
        said = wait_for_keys(store, [f"{key}/settings/{m}" for m in members], deadline,
                             "every bridge member's endpoint settings",
                             verdicts=[f"{key}/status/{m}" for m in members if m != rank])
        if len(set(said)) > 1:
            listed = "; ".join(f"rank {m}: {text}" for m, text in zip(members, said))
            raise ValueError(f"the leaders' verbs settings differ ({listed}); set the same GPUBRIDGE_VERBS_* "
                             "values on every leader")
        endpoint = _rdma.Endpoint.over_sockets(
            index, len(members),
            publish=lambda name: store.set(f"{key}/socket/{rank}", name),
            collect=lambda: wait_for_keys(store, [f"{key}/socket/{m}" for m in members], deadline,
                                          "every bridge member's socket name",
                                          verdicts=[f"{key}/status/{m}" for m in members if m != rank]),
            timeout=max(0.1, deadline - time.monotonic()), tcp_host=tcp_host, **settings)
        return cls(endpoint, members, rank, timeout, chunk)

    @classmethod
    def over_fabric(cls, fabric: "_rdma.MockFabric", members: Sequence[int], rank: int, *,
                    timeout: timedelta = timedelta(seconds=30), chunk_bytes: int = 1 << 20,
                    router: Router | None = None, staging_bytes: int | None = None,
                    piece_bytes: int | None = None, **endpoint_settings) -> "RdmaTransport":
        """The bridge of member ``rank`` over an in-process fabric (tests, the kit)."""
        endpoint = fabric.endpoint(list(members).index(rank), **endpoint_settings)
        staging = RegisteredStaging(endpoint, staging_bytes, pin=False if not torch.cuda.is_available() else None)
        return cls(endpoint, members, rank, timeout, chunk_bytes, router, staging, piece_bytes)

    # -- collectives ---------------------------------------------------------------------------------
    def all_reduce(self, tensor: torch.Tensor, op: str = "sum") -> None:
        if len(self.members) == 1 or tensor.numel() == 0:
            return
        self._carry(tensor, lambda view, number, deadline: self.worker.all_reduce(
            view.data_ptr(), view.numel(), DTYPE_CODES[view.dtype], OP_CODES[op],
            max(1, self.chunk_bytes // view.element_size()), number, deadline),
            where_it_lies=lambda flat, number, deadline: self._on_device(flat).all_reduce(
                flat, op, max(1, self.chunk_bytes // flat.element_size()), number, deadline))

    def broadcast(self, tensor: torch.Tensor, src: int) -> None:
        if len(self.members) == 1 or tensor.numel() == 0:
            return
        root = self.members.index(src)
        self._carry(tensor, lambda view, number, deadline: self.worker.broadcast(
            view.data_ptr(), view.numel() * view.element_size(), root, max(1, self.chunk_bytes),
            number, deadline), only_out=self.index != root, only_in=self.index == root,
            where_it_lies=lambda flat, number, deadline: self._on_device(flat).broadcast(
                flat, root, self.chunk_bytes, number, deadline))

    def _on_device(self, flat: torch.Tensor) -> OnDevice:
        """Message by message, reductions where the tensor lives: before every post the
        tensor's stream has finished its producers, after every receive the device's flush
        plan has run."""
        if flat.device.type != "cuda":
            return OnDevice(self.worker, len(self.members), self.index)
        stream = torch.cuda.current_stream(flat.device)
        flush = self.router.plan(flat.device.index or 0)
        return OnDevice(self.worker, len(self.members), self.index, settle=stream.synchronize,
                        landed=flush.after_receive)

    def _carry(self, tensor: torch.Tensor, run, only_out: bool = False, only_in: bool = False,
               where_it_lies=None) -> None:
        if tensor.dtype not in DTYPE_CODES:
            raise ValueError(f"the {self.name} bridge cannot carry {tensor.dtype}")
        route = self.router.route(tensor)
        self.last_route = route
        deadline = time.monotonic() + self.timeout
        began = time.perf_counter()
        try:
            if route.how == "in-place":
                self._calls += 1
                self._in_place(tensor.view(-1), self._calls, deadline, where_it_lies)
            elif route.how == "plain":
                self._calls += 1
                run(tensor, self._calls, deadline)
            else:
                self._bounce(tensor, run, deadline, only_out, only_in)
        except BaseException as failure:
            self.worker.abort()
            if self.observations is not None:
                self.observations.emit("bridge_call", bridge=self.name, member=self.index, nbytes=tensor.nbytes,
                                       route=route.how, failed=type(failure).__name__)
            raise
        if self.observations is not None:
            self.observations.emit("bridge_call", bridge=self.name, member=self.index, nbytes=tensor.nbytes,
                                   route=route.how, ms=round((time.perf_counter() - began) * 1e3, 4))

    def _in_place(self, flat: torch.Tensor, number: int, deadline: float, where_it_lies) -> None:
        where_it_lies(flat, number, deadline)

    def _bounce(self, tensor: torch.Tensor, run, deadline: float, only_out: bool, only_in: bool) -> None:
        """Through registered host memory, in pieces: while the network works on piece ``i``
        the copy stream already brings piece ``i + 1`` to the host, and results go back to the
        device behind the network call.  Every piece is one numbered call, so both ends cut
        the tensor alike (the piece size is a setting all members share)."""
        flat = tensor.reshape(-1) if tensor.is_contiguous() else tensor.contiguous().view(-1)
        esize = flat.element_size()
        per_piece = max(1, self.piece_bytes // esize)
        pieces = [(lo, min(flat.numel(), lo + per_piece)) for lo in range(0, flat.numel(), per_piece)]
        on_gpu = flat.device.type == "cuda"
        if on_gpu and self._copy_stream is None:
            self._copy_stream = torch.cuda.Stream(flat.device)
        # two halves of one staging buffer, used alternately
        half = 1 << max(12, (per_piece * esize - 1).bit_length())
        stage = self.staging.take(2 * half)
        views = [stage[i * half:i * half + per_piece * esize].view(flat.dtype) for i in range(2)]
        landed = [None, None]

        def bring(i: int) -> None:
            lo, hi = pieces[i]
            host = views[i % 2][:hi - lo]
            if only_out:
                return
            if on_gpu:
                self._copy_stream.wait_stream(torch.cuda.current_stream(flat.device))
                with torch.cuda.stream(self._copy_stream):
                    host.copy_(flat[lo:hi], non_blocking=True)
                    landed[i % 2] = torch.cuda.Event()
                    landed[i % 2].record()
            else:
                host.copy_(flat[lo:hi])

        bring(0)
        for i, (lo, hi) in enumerate(pieces):
            host = views[i % 2][:hi - lo]
            if landed[i % 2] is not None:
                landed[i % 2].synchronize()
                landed[i % 2] = None
            if i + 1 < len(pieces):
                if on_gpu and not only_in:
                    # the other half still feeds the copy back of piece i - 1
                    self._copy_stream.synchronize()
                bring(i + 1)
            self._calls += 1
            run(host, self._calls, deadline)
            if only_in:
                continue
            if on_gpu:
                with torch.cuda.stream(self._copy_stream):
                    flat[lo:hi].copy_(host, non_blocking=True)
            else:
                flat[lo:hi].copy_(host)
        if on_gpu:
            torch.cuda.current_stream(flat.device).wait_stream(self._copy_stream)
            self._copy_stream.synchronize()          # the staging halves are free again
        if flat.data_ptr() != tensor.data_ptr() and not only_in:
            tensor.copy_(flat.view(tensor.shape))

    def describe(self) -> dict:
        return {"routes": dict(self.router.counts), "staging": {
            "held_bytes": self.staging.held_bytes(), "allocated": self.staging.allocated,
            "reused": self.staging.reused, "evicted": self.staging.evicted},
            "endpoint": self.worker.telemetry() if self.worker is not None else None}

    def close(self) -> None:
        if self.worker is not None:
            if self.observations is not None:
                try:
                    self.observations.emit("endpoint", **dict(self.worker.telemetry(), bridge=self.name, member=self.index))
                except Exception:  # noqa: BLE001 - a record less, never a failed close
                    pass
            self.staging.close()
        super().close()
