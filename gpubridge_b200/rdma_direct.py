"""Device memory an adapter reads and writes in place: the registrar of ``csrc/gb_direct.cpp``.

    registrar = Registrar.pretend()                    # pretend device memory and adapter (tests)
    registrar = Registrar.on_this_machine()            # the CUDA driver, loaded at run time
    with registrar.acquire(tensor.data_ptr(), tensor.nbytes) as region:
        ... post work with region.key ...              # region.method: "dma-buf" or "peer memory"
    window = registrar.expose(pointer, nbytes)         # one receive a peer may write into
    registrar.close_window(window)

A range is registered through a dma-buf where the device exports them, else through a
peer-memory kernel module, else not at all - and then :class:`NotDirect` carries every reason
and the bridge stages through host memory (:mod:`gpubridge_b200.rdma_transport` routes such
tensors to ``bounce``).  Registrations are cached under the identity of the ALLOCATION, rounded
out to 2 MiB inside it; the same address in a later allocation is another owner.  Nothing cached
is remotely writable: a peer writes only into windows made for one receive each.
(Reference: the verbs crate's direct.rs and gpu.rs.)
"""
from __future__ import annotations

import contextlib
import ctypes
import dataclasses
import json

from gpubridge_b200.ops import _lib

METHODS = {1: "dma-buf", 2: "peer memory"}
DMABUF_ENV = "GPUBRIDGE_VERBS_DMABUF"              # 0: never register through a dma-buf
PEER_MEMORY_ENV = "GPUBRIDGE_VERBS_PEER_MEMORY"    # 0: never register through a peer-memory module
#: what a pretend device or adapter can be told to refuse (``Registrar.fail``)
FAILURES = {"device dma-buf": 0, "device peer memory": 1, "export": 2, "adapter dma-buf": 3, "adapter pointer": 4}


class NotDirect(RuntimeError):
    """The range cannot be registered for direct access; the message lists every reason."""


@dataclasses.dataclass(frozen=True)
class Region:
    ticket: int
    method: str
    key: int
    lo: int
    hi: int


def _declare(lib) -> None:
    if getattr(lib, "_gb_direct_declared", False):
        return
    c, u64, ptr = ctypes, ctypes.c_ulonglong, ctypes.c_void_p
    table = {
        "gb_direct_new": (ptr, [c.c_int, c.c_char_p, u64]),
        "gb_direct_free": (None, [ptr]),
        "gb_direct_mock_alloc": (u64, [ptr, c.c_int, u64, u64]),
        "gb_direct_mock_release": (None, [ptr, u64]),
        "gb_direct_mock_fail": (None, [ptr, c.c_int, c.c_char_p]),
        "gb_direct_mock_counts": (None, [ptr, c.POINTER(u64)]),
        "gb_direct_acquire": (u64, [ptr, u64, u64, c.POINTER(c.c_int), c.POINTER(c.c_uint), c.POINTER(u64),
                                    c.POINTER(u64), c.c_char_p, c.c_size_t]),
        "gb_direct_release": (c.c_int, [ptr, u64]),
        "gb_direct_invalidate": (c.c_int, [ptr, u64, u64]),
        "gb_direct_expose": (u64, [ptr, u64, u64, c.POINTER(c.c_uint), c.c_char_p, c.c_size_t]),
        "gb_direct_close_window": (c.c_int, [ptr, u64]),
        "gb_direct_switch_off": (None, [ptr, c.c_int, c.c_char_p]),
        "gb_direct_capabilities": (None, [ptr, c.c_int, c.c_char_p, c.c_size_t]),
        "gb_direct_telemetry": (None, [ptr, c.c_char_p, c.c_size_t]),
    }
    for name, (restype, argtypes) in table.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = restype, argtypes
    lib._gb_direct_declared = True


class Registrar:
    def __init__(self, real: bool, modules_root: str = "", capacity: int = 64) -> None:
        self.lib = _lib.lib()
        _declare(self.lib)
        self.real = real
        self.handle = self.lib.gb_direct_new(1 if real else 0, modules_root.encode(), capacity)
        from gpubridge_b200 import config
        for method, name in ((1, DMABUF_ENV), (2, PEER_MEMORY_ENV)):      # GPUBRIDGE_VERBS_DMABUF=0 and the like
            if config._raw(name) and not config.flag(name):
                self.switch_off(METHODS[method], f"switched off by {name}")

    def switch_off(self, method: str, reason: str = "switched off") -> None:
        """Never try ``method`` ("dma-buf" or "peer memory"); an empty reason switches it back on."""
        code = {name: number for number, name in METHODS.items()}[method]
        self.lib.gb_direct_switch_off(self.handle, code, reason.encode())

    @classmethod
    def pretend(cls, modules_root: str = "", capacity: int = 64) -> "Registrar":
        """Pretend device memory (``alloc`` / ``free``) and a pretend adapter; ``modules_root`` is
        where ``proc/modules`` is read from, so a test decides whether a peer-memory module is loaded."""
        return cls(False, modules_root, capacity)

    @classmethod
    def on_this_machine(cls, capacity: int = 64) -> "Registrar":
        return cls(True, "", capacity)

    # -- the pretend device
    def alloc(self, size: int, device: int = 0, at: int = 0) -> int:
        return self.lib.gb_direct_mock_alloc(self.handle, device, size, at)

    def free(self, pointer: int) -> None:
        self.lib.gb_direct_mock_release(self.handle, pointer)

    def fail(self, what: str, reason: str = "") -> None:
        self.lib.gb_direct_mock_fail(self.handle, FAILURES[what], reason.encode())

    def counts(self) -> dict:
        six = (ctypes.c_ulonglong * 6)()
        self.lib.gb_direct_mock_counts(self.handle, six)
        names = ("exports", "descriptors_open", "descriptors_closed_twice", "registrations_alive",
                 "registrations_made", "registrations_released")
        return dict(zip(names, (int(v) for v in six)))

    # -- registrations
    def take(self, pointer: int, nbytes: int) -> Region:
        method, key = ctypes.c_int(), ctypes.c_uint()
        lo, hi = ctypes.c_ulonglong(), ctypes.c_ulonglong()
        why = ctypes.create_string_buffer(1024)
        ticket = self.lib.gb_direct_acquire(self.handle, pointer, nbytes, ctypes.byref(method), ctypes.byref(key),
                                            ctypes.byref(lo), ctypes.byref(hi), why, len(why))
        if not ticket:
            raise NotDirect(why.value.decode())
        return Region(ticket, METHODS[method.value], key.value, lo.value, hi.value)

    def give_back(self, region: Region) -> None:
        if self.lib.gb_direct_release(self.handle, region.ticket) != 0:
            raise ValueError("this registration was given back already")

    @contextlib.contextmanager
    def acquire(self, pointer: int, nbytes: int):
        region = self.take(pointer, nbytes)
        try:
            yield region
        finally:
            self.give_back(region)

    def invalidate(self, pointer: int, nbytes: int) -> int:
        """The owner is about to free the range; returns how many cached registrations overlapped it."""
        return self.lib.gb_direct_invalidate(self.handle, pointer, nbytes)

    def expose(self, pointer: int, nbytes: int) -> tuple[int, int]:
        """(window, remote key) for one receive of exactly these bytes."""
        key = ctypes.c_uint()
        why = ctypes.create_string_buffer(1024)
        window = self.lib.gb_direct_expose(self.handle, pointer, nbytes, ctypes.byref(key), why, len(why))
        if not window:
            raise NotDirect(why.value.decode())
        return window, key.value

    def close_window(self, window: int) -> None:
        if self.lib.gb_direct_close_window(self.handle, window) != 0:
            raise ValueError("no such window")

    def capabilities(self, device: int = 0) -> str:
        text = ctypes.create_string_buffer(1024)
        self.lib.gb_direct_capabilities(self.handle, device, text, len(text))
        return text.value.decode()

    def telemetry(self) -> dict:
        text = ctypes.create_string_buffer(1024)
        self.lib.gb_direct_telemetry(self.handle, text, len(text))
        return json.loads(text.value.decode())

    def close(self) -> None:
        handle, self.handle = self.handle, None
        if handle:
            self.lib.gb_direct_free(handle)
