"""``bridge="multitcp"``: the tagged bridge over the native multi-stream TCP worker.

The worker is ``csrc/gb_tcp.cpp`` inside the library (the reference ships it as a Rust crate
with the same C ABI idea: src/gpubridge/multitcp/__init__.py, crate/src/lib.rs).  Settings:
``GPUBRIDGE_MULTITCP_STREAMS`` (connections per peer, default 4),
``GPUBRIDGE_MULTITCP_CHUNK_BYTES`` (default 4 MiB), ``GPUBRIDGE_MULTITCP_IFADDR`` (the
local IPv4 address to listen on) or ``GPUBRIDGE_MULTITCP_IFNAME`` (an interface name, as in
the reference); default 127.0.0.1 for one box.

``python -m gpubridge_b200.multitcp info`` prints the protocol version and the settings.
"""
from __future__ import annotations

import ctypes
import json
import os
import sys
import time

from gpubridge_b200 import config as _config
from gpubridge_b200.tagged import Guarded, TaggedBridge, wait_for_keys
from gpubridge_b200.transport import register_transport

STREAMS_ENV = "GPUBRIDGE_MULTITCP_STREAMS"
CHUNK_ENV = "GPUBRIDGE_MULTITCP_CHUNK_BYTES"
IFADDR_ENV = "GPUBRIDGE_MULTITCP_IFADDR"
IFNAME_ENV = "GPUBRIDGE_MULTITCP_IFNAME"          # the reference's way to name the interface


def listen_address() -> str:
    """The local IPv4 address the worker listens on: ``GPUBRIDGE_MULTITCP_IFADDR``, else the
    first IPv4 address of the interface named by ``GPUBRIDGE_MULTITCP_IFNAME``, else loopback."""
    address = os.environ.get(IFADDR_ENV, "").strip()
    if address:
        return address
    name = os.environ.get(IFNAME_ENV, "").strip()
    if name:
        import socket

        import psutil
        for entry in psutil.net_if_addrs().get(name, []):
            if entry.family == socket.AF_INET:
                return entry.address
        raise ValueError(f"{IFNAME_ENV}={name}: no such interface with an IPv4 address here")
    return "127.0.0.1"


def _library():
    from gpubridge_b200.ops import _lib
    L = _lib.lib()
    if not getattr(L, "_tcp_declared", False):
        vp, i, u64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_uint64
        L.gb_tcp_create.restype = vp
        L.gb_tcp_create.argtypes = [i, i, i, ctypes.c_char_p]
        L.gb_tcp_address.argtypes = [vp, ctypes.c_char_p, i]
        L.gb_tcp_connect.argtypes = [vp, ctypes.POINTER(ctypes.c_char_p), ctypes.c_double]
        L.gb_tcp_send.restype = ctypes.c_long
        L.gb_tcp_send.argtypes = [vp, i, vp, u64, u64]
        L.gb_tcp_recv.restype = ctypes.c_long
        L.gb_tcp_recv.argtypes = [vp, i, vp, u64, u64]
        L.gb_tcp_wait.argtypes = [vp, ctypes.POINTER(ctypes.c_long), i, ctypes.c_double]
        L.gb_tcp_all_reduce.argtypes = [vp, vp, u64, i, i, u64, u64, ctypes.c_double]
        L.gb_tcp_broadcast.argtypes = [vp, vp, u64, i, u64, u64, ctypes.c_double]
        L.gb_tcp_abort.argtypes = [vp]
        L.gb_tcp_close.argtypes = [vp]
        L.gb_tcp_last_error.restype = ctypes.c_char_p
        L.gb_tcp_last_error.argtypes = [vp]
        L._tcp_declared = True
    return L


def streams_setting() -> int:
    raw = os.environ.get(STREAMS_ENV, "").strip()
    value = int(raw) if raw else 4
    if not 1 <= value <= 64:
        raise ValueError(f"{STREAMS_ENV} must be between 1 and 64")
    return value


class Worker(Guarded):
    """One member's native worker.  Calls from several threads are counted, so that ``close``
    frees the worker only after every one of them has left the library."""

    _what = "multitcp"

    def __init__(self, index: int, members: int, streams: int, host: str) -> None:
        self._guard()
        self.lib = _library()
        self.handle = self.lib.gb_tcp_create(index, members, streams, host.encode())
        if not self.handle:
            raise RuntimeError(f"multitcp: {self.lib.gb_tcp_last_error(None).decode()}")

    def _fail(self, handle: int):
        raise RuntimeError(f"multitcp: {self.lib.gb_tcp_last_error(handle).decode()}")

    def address(self) -> str:
        buf = ctypes.create_string_buffer(128)
        with self._inside() as handle:
            self.lib.gb_tcp_address(handle, buf, 128)
        return buf.value.decode()

    def connect(self, addresses: list[str], timeout_s: float) -> None:
        array = (ctypes.c_char_p * len(addresses))(*[a.encode() for a in addresses])
        with self._inside() as handle:
            if self.lib.gb_tcp_connect(handle, array, timeout_s) != 0:
                self._fail(handle)

    def send(self, peer: int, ptr: int, nbytes: int, tag: int) -> int:
        with self._inside() as handle:
            op = self.lib.gb_tcp_send(handle, peer, ptr, nbytes, tag)
            if op < 0:
                self._fail(handle)
            return op

    def recv(self, peer: int, ptr: int, nbytes: int, tag: int) -> int:
        with self._inside() as handle:
            op = self.lib.gb_tcp_recv(handle, peer, ptr, nbytes, tag)
            if op < 0:
                self._fail(handle)
            return op

    def wait(self, ids: list[int], deadline: float) -> None:
        array = (ctypes.c_long * len(ids))(*ids)
        left = max(0.001, deadline - time.monotonic())
        with self._inside() as handle:
            if self.lib.gb_tcp_wait(handle, array, len(ids), left) != 0:
                self._fail(handle)

    # The collectives themselves run inside the library (csrc/gb_tcp.cpp): chunked, pipelined,
    # in the reduction order tagged.py documents, without a Python round trip per chunk.
    def all_reduce(self, ptr: int, count: int, dtype: int, op: int, chunk_elems: int, seq: int,
                   deadline: float) -> None:
        left = max(0.001, deadline - time.monotonic())
        with self._inside() as handle:
            if self.lib.gb_tcp_all_reduce(handle, ptr, count, dtype, op, chunk_elems, seq, left) != 0:
                self._fail(handle)

    def broadcast(self, ptr: int, nbytes: int, root: int, chunk_bytes: int, seq: int,
                  deadline: float) -> None:
        left = max(0.001, deadline - time.monotonic())
        with self._inside() as handle:
            if self.lib.gb_tcp_broadcast(handle, ptr, nbytes, root, chunk_bytes, seq, left) != 0:
                self._fail(handle)

    def abort(self) -> None:
        try:
            with self._inside() as handle:
                self.lib.gb_tcp_abort(handle)
        except RuntimeError:
            pass                                           # closed already

    def close(self) -> None:
        self._retire(self.lib.gb_tcp_abort, self.lib.gb_tcp_close)


@register_transport
class MultiTcpTransport(TaggedBridge):
    name = "multitcp"

    @classmethod
    def _connect(cls, store, key, members, rank, timeout, deadline):
        index = members.index(rank)
        host = listen_address()
        chunk = _config.size_setting(CHUNK_ENV, 4 << 20)
        streams = streams_setting()
        worker = Worker(index, len(members), streams, host)
        try:
            # the address travels with the settings both ends of a link must share: the lower
            # member dials `streams` connections and the higher one waits for exactly as many
            mine = json.dumps({"address": worker.address(), "streams": streams, "chunk_bytes": chunk})
            store.set(f"{key}/address/{rank}", mine)
            said = [json.loads(text) for text in wait_for_keys(
                store, [f"{key}/address/{m}" for m in members], deadline, "every bridge member's multitcp address",
                verdicts=[f"{key}/status/{m}" for m in members if m != rank])]
            for name, variable in (("streams", STREAMS_ENV), ("chunk_bytes", CHUNK_ENV)):
                values = {m: told[name] for m, told in zip(members, said)}
                if len(set(values.values())) > 1:
                    listed = ", ".join(f"rank {m}: {v}" for m, v in values.items())
                    raise ValueError(f"{variable} differs between the leaders ({listed}); set the same value on each")
            worker.connect([told["address"] for told in said], max(0.1, deadline - time.monotonic()))
            return cls(worker, members, rank, timeout, chunk)
        except BaseException:
            worker.close()
            raise


def main(argv: list[str]) -> int:
    command = argv[0] if argv else "info"
    if command == "build":
        from gpubridge_b200.ops import _build
        print(_build.build())
        return 0
    if command == "info":
        print(json.dumps({"protocol": _library().gb_tcp_protocol(), "streams": streams_setting(),
                          "chunk_bytes": _config.size_setting(CHUNK_ENV, 4 << 20),
                          "ifaddr": listen_address()}))
        return 0
    print("usage: python -m gpubridge_b200.multitcp [build|info]", file=sys.stderr)
    return 2


if __name__ == "__main__":
    sys.exit(main(sys.argv[1:]))
