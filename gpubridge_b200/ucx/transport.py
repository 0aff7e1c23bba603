"""``bridge="ucx"``: the island leaders' bridge over UCX tagged messages.

UCX picks what carries the bytes (InfiniBand or RoCE verbs, shared memory, TCP).  Per tensor
the bridge takes one of three paths and records it in :attr:`UcxTransport.last_path`:

``host``    a contiguous host tensor: the worker's native collectives run on it as it lies
            (chunked exchange for two leaders, ring for more, root-sends broadcast);
``direct``  a device tensor, when this rank's UCX was built with CUDA memory support and the
            device's direct writes can be made visible (:mod:`gpubridge_b200.gdr`): UCX reads and
            writes the device memory itself, the reductions run on the device, message by
            message (:class:`gpubridge_b200.tagged.OnDevice`), each step after the tensor's stream has
            finished and each receive followed by the device's flush;
``staged``  every other device tensor, and non-contiguous ones: through pinned host memory in
            pieces, the device copy of piece ``i + 1`` overlapping the network's piece ``i``.

Link set-up is collective over the job: every leader publishes its worker address with its UCX
version and chunk size; leaders whose UCX versions (major.minor) or chunk sizes differ refuse
the link, and - like a leader whose UCX did not start - make ``init`` fail with the same message
on every rank.  Every wait has the deadline ``init`` gave its groups; after a timeout or a lost
peer the transport refuses later calls.  (Reference: src/gpubridge/ucx/transport.py.)
"""
from __future__ import annotations

import base64
import json
import time
from datetime import timedelta
from typing import Sequence

import torch

from gpubridge_b200 import config as _config
from gpubridge_b200 import ucx as _ucx
from gpubridge_b200.rdma_transport import RdmaTransport, RegisteredStaging, Route, Router
from gpubridge_b200.tagged import wait_for_keys

CHUNK_ENV = "GPUBRIDGE_UCX_CHUNK_BYTES"
DIRECT_MIN_ENV = "GPUBRIDGE_UCX_DIRECT_MIN_BYTES"
PATHS = {"plain": "host", "in-place": "direct", "bounce": "staged"}


def chunk_bytes_setting() -> int:
    return _config.size_setting(CHUNK_ENV, 4 << 20, multiple=8)


def choose_path(device_type: str, contiguous: bool, memory_types: set[str], direct_ok: bool = True) -> str:
    """The path of a tensor (see the module text), from facts alone."""
    if not contiguous:
        return "staged"
    if device_type == "cpu":
        return "host"
    return "direct" if "cuda" in memory_types and direct_ok else "staged"


class UcxTransport(RdmaTransport):
    name = "ucx"
    device_tensors = True
    _instead = 'use bridge="multitcp" or bridge="gloo" across machines'

    def __init__(self, worker, members: Sequence[int], rank: int, timeout: timedelta, chunk_bytes: int,
                 router: Router | None = None, staging: RegisteredStaging | None = None,
                 piece_bytes: int | None = None) -> None:
        if router is None:
            router = Router(device_registration="cuda" in worker.memory_types(),
                            direct_min_bytes=_config.size_setting(DIRECT_MIN_ENV, 0, multiple=1))
        super().__init__(worker, members, rank, timeout, chunk_bytes, router,
                         staging or RegisteredStaging(worker), piece_bytes)

    @property
    def last_path(self) -> str | None:
        return PATHS[self.last_route.how] if self.last_route is not None else None

    @property
    def flush_method(self) -> str:
        """How direct receives are made visible on the device of the last direct call."""
        device = torch.cuda.current_device() if torch.cuda.is_available() else 0
        return self.router.plan(device).reason

    @classmethod
    def _connect(cls, store, key, members, rank, timeout, deadline):
        index = list(members).index(rank)
        chunk = chunk_bytes_setting()                 # a bad setting fails here, on this leader
        worker = _ucx.Worker(len(members), index)
        try:
            mine = {"address": base64.b64encode(worker.address()).decode(), "chunk": chunk,
                    "version": list(_ucx.version())}
            store.set(f"{key}/hello/{rank}", json.dumps(mine))
            said = [json.loads(text) for text in wait_for_keys(
                store, [f"{key}/hello/{m}" for m in members], deadline, "every leader's UCX address",
                verdicts=[f"{key}/status/{m}" for m in members if m != rank])]
            versions = {m: tuple(s["version"][:2]) for m, s in zip(members, said)}
            if len(set(versions.values())) > 1:
                listed = ", ".join(f"rank {m}: {'.'.join(map(str, v))}" for m, v in versions.items())
                raise _ucx.UcxError(f"the leaders run different UCX versions ({listed}); their wire "
                                    "protocols are not promised to match")
            chunks = {m: s["chunk"] for m, s in zip(members, said)}
            if len(set(chunks.values())) > 1:
                listed = ", ".join(f"rank {m}: {c}" for m, c in chunks.items())
                raise _ucx.UcxError(f"{CHUNK_ENV} differs between the leaders ({listed}); both ends "
                                    "of a link must cut messages alike")
            for member, told in enumerate(said):
                if member != index:
                    worker.connect(member, base64.b64decode(told["address"]))
            return cls(worker, members, rank, timeout, chunk)
        except BaseException:
            worker.close(2.0)
            raise

    def _in_place(self, flat: torch.Tensor, number: int, deadline: float, where_it_lies) -> None:
        on_gpu = flat.device.type == "cuda"
        self.worker.memory(_ucx.CUDA if on_gpu else _ucx.HOST)
        try:
            where_it_lies(flat, number, deadline)
        finally:
            if self.worker is not None and self.worker.handle:
                self.worker.memory(_ucx.HOST)

    @classmethod
    def create_p2p(cls, group, *, store=None, timeout=None):
        """The wire of the cross-island point-to-point engine: workers of its own, one per peer."""
        from gpubridge_b200.tagged import DEFAULT_TIMEOUT
        from gpubridge_b200.ucx.p2p import UcxLink
        return UcxLink(group.rank, store, timeout or DEFAULT_TIMEOUT)

    def describe(self) -> dict:
        told = super().describe()
        told["paths"] = {PATHS[how]: count for how, count in self.router.counts.items()}
        return told


def load(name: str) -> None:
    """Called when ``bridge="ucx"`` is resolved: compiles and loads the worker (or says why it
    cannot, on every rank alike) and registers the transport."""
    _ucx.load()
    from gpubridge_b200 import transport
    transport.register_transport(UcxTransport)
