"""The RDMA-style tagged endpoint (``csrc/gb_rdma.cpp``) from Python, and ``bridge="verbs"``.

The endpoint is the host-staged bridge for links made of reliable connected queue pairs
(InfiniBand / RoCE): eager messages through pre-posted, credit-controlled receive slots,
large ones by rendezvous - the receiver registers the user's buffer (an LRU cache of
registrations), grants it, the sender writes into it and says when it is done.  It is written
against a provider interface.  Two things can be had here:

* :class:`MockFabric` / :class:`Endpoint`: the whole protocol over an in-process fabric that can
  be told to fail, drop, delay or corrupt an operation or kill a member - how the protocol,
  its flow control and its failure rule are tested, without a NIC;
* the name ``bridge="verbs"``.  A provider over libibverbs needs headers this image does not
  have, so none is built, and resolving the name raises - on every rank alike, before anything
  is connected - an error that says so: the behaviour the reference has where its shim cannot
  be built (src/gpubridge/verbs/__init__.py:63-64).

Settings an endpoint takes (0 keeps the default): ``eager_max`` (16 KiB; larger messages go by
rendezvous), ``data_slots`` / ``ctrl_slots`` (16 / 8 receive slots per peer and class),
``max_write`` (1 MiB per one-sided write), ``unexpected_max`` (64 MiB of early eager messages),
``mr_cache`` (64 registrations).  :meth:`Endpoint.telemetry` returns the counters as a dict.
"""
from __future__ import annotations

import ctypes
import json
import time


FAULTS = {"error": 1, "drop": 2, "delay": 3, "corrupt": 4, "kill": 5, "spurious": 6, "late": 7}
OPCODES = {"send": 0, "write": 2, "any": -1}


def _library():
    from gpubridge_b200.ops import _lib
    L = _lib.lib()
    if not getattr(L, "_rdma_declared", False):
        vp, i, u64, u = ctypes.c_void_p, ctypes.c_int, ctypes.c_ulonglong, ctypes.c_uint
        L.gb_rdma_mock_fabric.restype = vp
        L.gb_rdma_mock_fabric.argtypes = [i]
        L.gb_rdma_mock_free.restype = None
        L.gb_rdma_mock_free.argtypes = [vp]
        L.gb_rdma_mock_inject.restype = None
        L.gb_rdma_mock_inject.argtypes = [vp, i, i, i, i, ctypes.c_long, i]
        L.gb_rdma_mock_stats.restype = ctypes.c_char_p
        L.gb_rdma_mock_stats.argtypes = [vp]
        L.gb_rdma_create.restype = vp
        L.gb_rdma_create.argtypes = [vp, i, u, u, u, u, u64, u]
        for name in ("gb_rdma_send", "gb_rdma_recv"):
            getattr(L, name).restype = ctypes.c_long
            getattr(L, name).argtypes = [vp, i, vp, u64, u64]
        L.gb_rdma_wait.argtypes = [vp, ctypes.POINTER(ctypes.c_long), i, ctypes.c_double]
        L.gb_rdma_all_reduce.argtypes = [vp, vp, u64, i, i, u64, u64, ctypes.c_double]
        L.gb_rdma_broadcast.argtypes = [vp, vp, u64, i, u64, u64, ctypes.c_double]
        L.gb_rdma_invalidate.argtypes = [vp, vp, u64]
        for name in ("gb_rdma_last_error", "gb_rdma_telemetry"):
            getattr(L, name).restype = ctypes.c_char_p
            getattr(L, name).argtypes = [vp]
        L.gb_rdma_abort.restype = L.gb_rdma_close.restype = None
        L.gb_rdma_abort.argtypes = L.gb_rdma_close.argtypes = [vp]
        L.gb_rdma_socket_provider.restype = vp
        L.gb_rdma_socket_provider.argtypes = [i, i, ctypes.c_char_p]
        L.gb_rdma_socket_connect.argtypes = [vp, ctypes.POINTER(ctypes.c_char_p), ctypes.c_double]
        L.gb_rdma_socket_error.restype = ctypes.c_char_p
        L.gb_rdma_socket_name.restype = ctypes.c_char_p
        L.gb_rdma_socket_name.argtypes = [vp]
        L.gb_rdma_socket_free.restype = None
        L.gb_rdma_socket_free.argtypes = [vp]
        L.gb_rdma_create_on.restype = vp
        L.gb_rdma_create_on.argtypes = [vp, u, u, u, u, u64, u]
        L._rdma_declared = True
    return L


def protocol_version() -> int:
    return _library().gb_rdma_protocol()


from gpubridge_b200.tagged import Guarded as _Guarded  # noqa: E402


class MockFabric:
    """``members`` connected members inside this process."""

    def __init__(self, members: int) -> None:
        self.lib, self.members = _library(), members
        self.handle = self.lib.gb_rdma_mock_fabric(members)
        if not self.handle:
            raise ValueError("a mock fabric has 1 to 64 members")
        self.endpoints: list[Endpoint] = []

    def endpoint(self, index: int, **settings) -> "Endpoint":
        made = Endpoint(self, index, **settings)
        self.endpoints.append(made)
        return made

    def inject(self, fault: str, *, src: int = -1, dst: int = -1, on: str = "any", nth: int = 1,
               milliseconds: int = 0) -> None:
        """The ``nth`` next operation of kind ``on`` (send / write / any) from ``src`` to ``dst``
        (-1: any) will ``error``, ``drop``, ``delay``, be ``corrupt`` or ``kill`` its destination;
        ``spurious``: both ends' polls wake ``milliseconds`` times with nothing to report and the
        operation goes through; ``late``: it is carried out at once but its completion reaches
        the poster ``milliseconds`` later, so the peer's answer may overtake it."""
        self.lib.gb_rdma_mock_inject(self.handle, FAULTS[fault], src, dst, OPCODES[on], nth, milliseconds)

    def stats(self) -> dict:
        return json.loads(self.lib.gb_rdma_mock_stats(self.handle).decode())

    def close(self) -> None:
        for endpoint in self.endpoints:
            endpoint.close()
        handle, self.handle = self.handle, None
        if handle:
            self.lib.gb_rdma_mock_free(handle)


class Endpoint(_Guarded):
    """One member's endpoint; the worker interface :class:`~gpubridge_b200.tagged.TaggedBridge`
    expects (``all_reduce`` / ``broadcast`` / ``abort`` / ``close``) plus send / recv / wait."""

    def __init__(self, fabric: "MockFabric | None", index: int, *, eager_max: int = 0, data_slots: int = 0,
                 ctrl_slots: int = 0, max_write: int = 0, unexpected_max: int = 0, mr_cache: int = 0,
                 _handle: int | None = None) -> None:
        self._guard()
        if _handle is not None:                           # an endpoint made elsewhere (over_sockets)
            self.lib, self.index, self.handle = _library(), index, _handle
            return
        self.lib, self.index = fabric.lib, index
        self.handle = self.lib.gb_rdma_create(fabric.handle, index, eager_max, data_slots, ctrl_slots,
                                              max_write, unexpected_max, mr_cache)
        if not self.handle:
            raise ValueError(f"member {index} is not on this fabric")

    @classmethod
    def over_sockets(cls, index: int, members: int, publish, collect, timeout: float = 60.0, *,
                     tcp_host: str | None = None, eager_max: int = 0, data_slots: int = 0, ctrl_slots: int = 0, max_write: int = 0,
                     unexpected_max: int = 0, mr_cache: int = 0) -> "Endpoint":
        """Member ``index`` of ``members`` processes on one host, joined by Unix-domain sockets
        (the socket provider of ``csrc/gb_rdma.cpp``: the endpoint's whole protocol between
        processes, where no adapter exists).  ``publish(name)`` makes this member's socket name
        known; ``collect()`` returns every member's, in member order (a store does both).
        ``tcp_host``: listen on that IPv4 address with TCP instead (a port the system picks), so
        the members may sit on different hosts."""
        import os
        import uuid
        lib = _library()
        name = (f"tcp://{tcp_host}:0" if tcp_host else
                f"gpubridge-rdma-{os.getpid()}-{uuid.uuid4().hex[:12]}-{index}")
        provider = lib.gb_rdma_socket_provider(index, members, name.encode())
        if not provider:
            raise RuntimeError(f"rdma endpoint: could not listen on {name}")
        try:
            name = lib.gb_rdma_socket_name(provider).decode()
            publish(name)
            names = collect()
            array = (ctypes.c_char_p * members)(*[n.encode() for n in names])
            if lib.gb_rdma_socket_connect(provider, array, timeout) != 0:
                raise RuntimeError(f"rdma endpoint: {lib.gb_rdma_socket_error().decode()}")
        except BaseException:
            lib.gb_rdma_socket_free(provider)
            raise
        handle = lib.gb_rdma_create_on(provider, eager_max, data_slots, ctrl_slots, max_write,
                                       unexpected_max, mr_cache)
        return cls(None, index, _handle=handle)

    _what = "rdma endpoint"

    def _error(self, handle: int) -> str:
        return self.lib.gb_rdma_last_error(handle).decode()

    def last_error(self) -> str:
        """Why the endpoint broke (empty while it has not)."""
        with self._inside() as handle:
            return self._error(handle)

    def send(self, peer: int, ptr: int, nbytes: int, tag: int) -> int:
        with self._inside() as handle:
            op = self.lib.gb_rdma_send(handle, peer, ptr, nbytes, tag)
            if op < 0:
                raise RuntimeError(f"rdma endpoint: {self._error(handle) or 'no such peer'}")
            return op

    def recv(self, peer: int, ptr: int, nbytes: int, tag: int) -> int:
        with self._inside() as handle:
            op = self.lib.gb_rdma_recv(handle, peer, ptr, nbytes, tag)
            if op < 0:
                raise RuntimeError(f"rdma endpoint: {self._error(handle) or 'no such peer'}")
            return op

    def wait(self, ids: list[int], deadline: float) -> None:
        array = (ctypes.c_long * len(ids))(*ids)
        with self._inside() as handle:
            if self.lib.gb_rdma_wait(handle, array, len(ids), max(0.001, deadline - time.monotonic())) != 0:
                raise RuntimeError(f"rdma endpoint: {self._error(handle)}")

    def all_reduce(self, ptr: int, count: int, dtype: int, op: int, chunk_elems: int, seq: int,
                   deadline: float) -> None:
        left = max(0.001, deadline - time.monotonic())
        with self._inside() as handle:
            if self.lib.gb_rdma_all_reduce(handle, ptr, count, dtype, op, chunk_elems, seq, left) != 0:
                raise RuntimeError(f"rdma endpoint: {self._error(handle)}")

    def broadcast(self, ptr: int, nbytes: int, root: int, chunk_bytes: int, seq: int, deadline: float) -> None:
        left = max(0.001, deadline - time.monotonic())
        with self._inside() as handle:
            if self.lib.gb_rdma_broadcast(handle, ptr, nbytes, root, chunk_bytes, seq, left) != 0:
                raise RuntimeError(f"rdma endpoint: {self._error(handle)}")

    def invalidate(self, ptr: int, nbytes: int) -> int:
        """Forget cached registrations overlapping the range (call before freeing memory that
        large messages were received into); returns how many were dropped.  Nothing to forget
        on an endpoint that is closed already."""
        try:
            with self._inside() as handle:
                return self.lib.gb_rdma_invalidate(handle, ptr, nbytes)
        except RuntimeError:
            return 0

    def telemetry(self) -> dict:
        with self._inside() as handle:
            return json.loads(self.lib.gb_rdma_telemetry(handle).decode())

    def abort(self) -> None:
        try:
            with self._inside() as handle:
                self.lib.gb_rdma_abort(handle)
        except RuntimeError:
            pass                                           # closed already: nothing left to stop

    def close(self) -> None:
        """Leave in good order - unless other threads are still inside calls: those are ended
        first (their waits return with an error) and the endpoint is freed once they have left."""
        self._retire(self.lib.gb_rdma_abort, self.lib.gb_rdma_close)


PROVIDER_ENV = "GPUBRIDGE_VERBS_PROVIDER"


def provider_available() -> bool:
    """Whether ``bridge="verbs"`` can connect members here.  No provider over real queue pairs
    is part of this build (see the module text); ``GPUBRIDGE_VERBS_PROVIDER=sockets`` selects
    the socket provider over Unix-domain sockets, which joins the processes of ONE host, and
    ``=tcp`` the same provider over TCP (listening where ``GPUBRIDGE_MULTITCP_IFADDR`` /
    ``GPUBRIDGE_MULTITCP_IFNAME`` say, loopback otherwise), which joins hosts - the bridge's
    whole protocol end to end without an adapter, not a fast path."""
    return provider_kind() in ("sockets", "tcp")


def provider_kind() -> str:
    import os
    return os.environ.get(PROVIDER_ENV, "").strip().lower()


def load(name: str) -> None:
    """Called when ``bridge="verbs"`` is resolved: says, on every rank alike and before anything
    is connected, why the bridge cannot be used here."""
    if provider_available():
        from gpubridge_b200 import rdma_transport, transport
        transport.register_transport(rdma_transport.RdmaTransport)
        return
    raise ImportError(
        "the verbs bridge needs a provider over libibverbs, and this build has none: the "
        "infiniband/verbs.h header is not installed here.  The endpoint itself - wire protocol, "
        "flow control, registration cache, failure rule - is built and runs over an in-process "
        "fabric (gpubridge_b200.rdma.MockFabric) and, between the processes of one host, over "
        "Unix-domain sockets (GPUBRIDGE_VERBS_PROVIDER=sockets); across machines use "
        "bridge='multitcp' or 'gloo'")


def _device_registration() -> str:
    """What the registrar of device memory finds on this machine (device 0), in its own words."""
    try:
        from gpubridge_b200.rdma_direct import Registrar
        registrar = Registrar.on_this_machine()
        try:
            return registrar.capabilities(0)
        finally:
            registrar.close()
    except Exception as failure:  # noqa: BLE001 - informational
        return f"unknown ({type(failure).__name__}: {failure})"


def info() -> dict:
    """What this build has of the verbs bridge (``python -m gpubridge_b200.rdma info``)."""
    import ctypes.util
    import os
    return {"protocol": protocol_version(), "provider": "libibverbs" if provider_available() else None,
            "libibverbs_found": ctypes.util.find_library("ibverbs") is not None,
            "verbs_header": os.path.exists("/usr/include/infiniband/verbs.h"),
            "in_process_fabric": True, "device_registration": _device_registration(),
            "defaults": {"eager_max": 16 << 10, "data_slots": 16, "ctrl_slots": 8, "max_write": 1 << 20,
                         "unexpected_max": 64 << 20, "mr_cache": 64}}


def main(argv: list[str]) -> int:
    import sys
    command = argv[0] if argv else "info"
    if command == "build":
        from gpubridge_b200.ops import _build
        print(_build.build())
        return 0
    if command == "info":
        print(json.dumps(info()))
        return 0
    print("usage: python -m gpubridge_b200.rdma [build|info]", file=sys.stderr)
    return 2


if __name__ == "__main__":
    import sys
    sys.exit(main(sys.argv[1:]))
