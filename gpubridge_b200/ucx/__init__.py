"""The UCX worker behind ``bridge="ucx"``: build it, load it, call it.

``gb_ucx.cpp`` beside this file is a C++ worker over UCX's UCP tagged messages (it is kept out of
``csrc/``, whose every file is part of the package's own library).  UCX is a system library,
so nothing of it is compiled with the package: ``python -m gpubridge_b200.ucx build`` compiles
the worker against the UCX of this machine, and :func:`load` does so at first use - with the
system C++ compiler, UCX found through ``UCX_HOME``, ``pkg-config ucx`` or the default include
path, into ``GPUBRIDGE_UCX_LIB_DIR`` (default ``~/.cache/gpubridge_b200``).  The file name
carries a digest of everything that could change the result (sources, flags, compiler, UCX's
version header, machine), because that directory is often shared by the nodes of a cluster
that do not share one UCX.  Without a compiler or UCX, :class:`Unavailable` says what is
missing; nothing else in the package needs this module.

The collectives (two-member exchange, ring, broadcast; chunked, with a deadline) run inside the
worker (``csrc/gb_tagged.cpp``, compiled in); :class:`Worker` also gives the single messages, which the
bridge uses where the reduction has to run on a device.
(Reference: src/gpubridge/ucx/__init__.py, whose collectives run in Python.)
"""
from __future__ import annotations

import contextlib
import ctypes
import hashlib
import logging
import os
import platform
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from collections.abc import Sequence
from pathlib import Path

from gpubridge_b200.tagged import Guarded

CSRC = Path(__file__).resolve().parent.parent / "csrc"
SOURCES = (Path(__file__).resolve().parent / "gb_ucx.cpp", CSRC / "gb_tagged.cpp")
HEADERS = (CSRC / "gb_tagged.h",)
LIB_DIR_ENV = "GPUBRIDGE_UCX_LIB_DIR"
UCX_HOME_ENV = "UCX_HOME"

HOST, CUDA, DETECT = 0, 1, -1
FAILED, TIMED_OUT, PEER_FAILED = -1, -2, -3

log = logging.getLogger("gpubridge_b200")
_lock = threading.Lock()
_libraries: dict[str, ctypes.CDLL] = {}


class Unavailable(ImportError):
    """The UCX worker cannot be built or loaded on this machine; the message says why."""


class UcxError(RuntimeError):
    """A UCX operation failed, timed out or lost its peer.  ``code`` is the worker's."""

    def __init__(self, message: str, code: int = FAILED) -> None:
        super().__init__(message)
        self.code = code


# ---- finding UCX ------------------------------------------------------------------------------------
def ucx_flags() -> tuple[list[str], list[str]]:
    """(compiler flags, linker flags) for the UCX of this machine."""
    home = os.environ.get(UCX_HOME_ENV, "").strip()
    if home:
        prefix = Path(home)
        if not (prefix / "include" / "ucp" / "api" / "ucp.h").is_file():
            raise Unavailable(f"{UCX_HOME_ENV}={home} has no include/ucp/api/ucp.h")
        libdir = next((prefix / d for d in ("lib", "lib64") if (prefix / d).is_dir()), prefix / "lib")
        return [f"-I{prefix / 'include'}"], [f"-L{libdir}", f"-Wl,-rpath,{libdir}", "-lucp", "-lucs"]
    if shutil.which("pkg-config") is not None:
        found = subprocess.run(["pkg-config", "--cflags", "--libs", "ucx"], capture_output=True, text=True)
        if found.returncode == 0:
            words = found.stdout.split()
            return [w for w in words if w.startswith("-I")], [w for w in words if not w.startswith("-I")]
    if Path("/usr/include/ucp/api/ucp.h").is_file():
        return [], ["-lucp", "-lucs"]
    raise Unavailable(
        "UCX was not found: no ucp/api/ucp.h under /usr/include, pkg-config knows no 'ucx', and "
        f"{UCX_HOME_ENV} is not set.  Install UCX with its headers (libucx-dev, or a module), or "
        f"point {UCX_HOME_ENV} at its prefix; until then use bridge='multitcp' or 'gloo' across "
        "machines and 'nvlink' inside one NVSwitch box")


def compiler() -> str | None:
    return os.environ.get("CXX") or shutil.which("c++") or shutil.which("g++")


def _version_header(cflags: Sequence[str]) -> bytes:
    for flag in [*cflags, "-I/usr/include"]:
        header = Path(flag[2:]) / "ucp" / "api" / "ucp_version.h"
        if header.is_file():
            return header.read_bytes()
    return b""


def library_path() -> Path:
    """Where the worker built from these sources, for this UCX, compiler and machine, lives."""
    cflags, ldflags = ucx_flags()
    cxx = compiler() or ""
    told = subprocess.run([cxx, "--version"], capture_output=True, text=True).stdout if cxx else ""
    digest = hashlib.sha256()
    for part in (*(p.read_bytes() for p in (*SOURCES, *HEADERS)), " ".join(cflags + ldflags).encode(),
                 told.encode(), _version_header(cflags), platform.machine().encode(),
                 " ".join(platform.libc_ver()).encode()):
        digest.update(part)
        digest.update(b"\0")
    base = Path(os.environ.get(LIB_DIR_ENV) or Path.home() / ".cache" / "gpubridge_b200")
    return base / f"libgpubridge_b200_ucx-{digest.hexdigest()[:16]}.so"


def build(*, force: bool = False) -> Path:
    """Compile the worker (once per sources and UCX) and return the library's path."""
    if not sys.platform.startswith("linux"):
        raise Unavailable(f"the UCX bridge is for Linux (this is {sys.platform})")
    cxx = compiler()
    if cxx is None:
        raise Unavailable("no C++ compiler (c++, g++ or $CXX) to build the UCX worker with")
    target = library_path()
    if target.exists() and not force:
        return target
    cflags, ldflags = ucx_flags()
    target.parent.mkdir(parents=True, exist_ok=True)
    # a private name first, then an atomic rename: ranks that build at once never see half a file
    fd, name = tempfile.mkstemp(prefix=target.name + ".", suffix=".part", dir=target.parent)
    os.close(fd)
    command = [cxx, "-std=c++17", "-O2", "-fPIC", "-shared", f"-I{CSRC}", *cflags,
               *(str(s) for s in SOURCES), "-o", name, *ldflags, "-lpthread"]
    done = subprocess.run(command, capture_output=True, text=True)
    if done.returncode != 0:
        Path(name).unlink(missing_ok=True)
        raise Unavailable("compiling the UCX worker failed:\n  " + " ".join(command) + "\n" + done.stderr[-4000:])
    Path(name).replace(target)
    return target


def _declare(lib: ctypes.CDLL) -> ctypes.CDLL:
    c = ctypes
    u64, ptr = c.c_ulonglong, c.c_void_p
    table = {
        "gb_ucx_version": (None, [c.POINTER(c.c_uint)] * 3),
        "gb_ucx_built_against": (c.c_uint, []),
        "gb_ucx_create": (ptr, [c.c_int, c.c_int, c.c_char_p, c.c_size_t]),
        "gb_ucx_memory_types": (c.c_int, [ptr, c.POINTER(u64)]),
        "gb_ucx_address": (c.c_int, [ptr, ptr, c.c_size_t, c.POINTER(c.c_size_t)]),
        "gb_ucx_connect": (c.c_int, [ptr, c.c_int, c.c_char_p]),
        "gb_ucx_set_memory": (None, [ptr, c.c_int]),
        "gb_ucx_send": (c.c_longlong, [ptr, c.c_int, ptr, u64, u64]),
        "gb_ucx_recv": (c.c_longlong, [ptr, ptr, u64, u64]),
        "gb_ucx_wait": (c.c_int, [ptr, c.POINTER(c.c_longlong), c.c_int, c.c_double]),
        "gb_ucx_poll": (c.c_int, [ptr, c.POINTER(c.c_longlong), c.c_int]),
        "gb_ucx_all_reduce": (c.c_int, [ptr, ptr, u64, c.c_int, c.c_int, u64, u64, c.c_double]),
        "gb_ucx_broadcast": (c.c_int, [ptr, ptr, u64, c.c_int, u64, u64, c.c_double]),
        "gb_ucx_abort": (None, [ptr]),
        "gb_ucx_last_error": (c.c_int, [ptr, c.c_char_p, c.c_size_t]),
        "gb_ucx_counters": (None, [ptr, c.POINTER(u64)]),
        "gb_ucx_close": (c.c_int, [ptr, c.c_double]),
    }
    for name, (restype, argtypes) in table.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = restype, argtypes
    return lib


def load(*, build_if_missing: bool = True) -> ctypes.CDLL:
    """The worker's library, compiled first if need be.  Raises :class:`Unavailable`."""
    with _lock:
        path = build() if build_if_missing else library_path()
        key = str(path)
        if key in _libraries:
            return _libraries[key]
        if not path.exists():
            raise Unavailable("the UCX worker is not built; run python -m gpubridge_b200.ucx build")
        try:
            lib = _declare(ctypes.CDLL(key))
        except OSError as first:
            if not build_if_missing:
                raise Unavailable(f"loading {path} failed: {first}") from None
            try:                                  # a damaged file in the cache: compile once more
                lib = _declare(ctypes.CDLL(str(build(force=True))))
            except OSError as second:
                raise Unavailable(f"loading {path} failed: {second}") from None
        _libraries[key] = lib
        return lib


def version() -> tuple[int, int, int]:
    """The version of the UCX library the worker RUNS with."""
    parts = [ctypes.c_uint() for _ in range(3)]
    load().gb_ucx_version(*(ctypes.byref(p) for p in parts))
    return tuple(p.value for p in parts)


def info() -> dict:
    """What is known about UCX here (``python -m gpubridge_b200.ucx info``); never raises."""
    out: dict = {"compiler": compiler(), UCX_HOME_ENV: os.environ.get(UCX_HOME_ENV) or None}
    try:
        cflags, ldflags = ucx_flags()
        out.update(found=True, cflags=cflags, ldflags=ldflags, library=str(library_path()),
                   built=library_path().exists())
    except Unavailable as why:
        out.update(found=False, why=str(why))
    return out


# ---- the worker -------------------------------------------------------------------------------------
class Worker(Guarded):
    """One UCP context and worker with an endpoint per other member.  Calls are serialised
    inside the library and counted here, so that ``close`` frees the worker only after every
    thread has left it; the object is the ``worker`` of a
    :class:`~gpubridge_b200.tagged.TaggedBridge`."""

    _what = "UCX"

    def __init__(self, members: int, index: int) -> None:
        self._guard()
        self.lib = load()
        self.members, self.index = members, index
        text = ctypes.create_string_buffer(512)
        self.handle = self.lib.gb_ucx_create(members, index, text, len(text))
        if not self.handle:
            raise UcxError(
                f"{text.value.decode()}.  UCX tries every transport it finds; where one of them "
                "cannot really be used (common on cloud machines), name the ones to use with "
                "UCX_TLS (tcp,self; rc,self on InfiniBand) or UCX_NET_DEVICES")

    @contextlib.contextmanager
    def _inside(self):
        try:
            with super()._inside() as handle:
                yield handle
        except RuntimeError as failure:
            if isinstance(failure, UcxError) or "is closed" not in str(failure):
                raise
            raise UcxError("the UCX worker is closed") from None

    # -- errors
    def _text(self, handle: int) -> str:
        text = ctypes.create_string_buffer(1024)
        self.lib.gb_ucx_last_error(handle, text, len(text))
        return text.value.decode(errors="replace")

    def last_error(self) -> str:
        with self._inside() as handle:
            return self._text(handle)

    def _check(self, handle: int, code: int) -> int:
        if code < 0:
            kind = {TIMED_OUT: "timed out", PEER_FAILED: "lost a peer"}.get(code, "failed")
            raise UcxError(f"UCX {kind}: {self._text(handle)}", code)
        return code

    # -- set-up
    def memory_types(self) -> set[str]:
        bits = ctypes.c_ulonglong()
        with self._inside() as handle:
            self._check(handle, self.lib.gb_ucx_memory_types(handle, ctypes.byref(bits)))
        return {name for name, bit in (("host", 1), ("cuda", 2)) if bits.value & bit}

    def address(self) -> bytes:
        room = 1024
        while True:
            buffer, length = ctypes.create_string_buffer(room), ctypes.c_size_t()
            with self._inside() as handle:
                code = self._check(handle, self.lib.gb_ucx_address(handle, buffer, room, ctypes.byref(length)))
            if code == 0:
                return buffer.raw[:length.value]
            room = length.value

    def connect(self, member: int, address: bytes) -> None:
        with self._inside() as handle:
            self._check(handle, self.lib.gb_ucx_connect(handle, member, address))

    # -- single messages
    def memory(self, kind: int) -> None:
        """Memory type of the buffers of the posts that follow (:data:`HOST`, :data:`CUDA`)."""
        with self._inside() as handle:
            self.lib.gb_ucx_set_memory(handle, kind)

    def send(self, member: int, pointer: int, nbytes: int, tag: int) -> int:
        with self._inside() as handle:
            return self._check(handle, self.lib.gb_ucx_send(handle, member, pointer, nbytes, tag))

    def recv(self, member: int, pointer: int, nbytes: int, tag: int) -> int:
        """``member`` is for the reader: a UCX receive names no peer, the tag says whose message it is."""
        with self._inside() as handle:
            return self._check(handle, self.lib.gb_ucx_recv(handle, pointer, nbytes, tag))

    def wait(self, ids: Sequence[int], deadline: float) -> None:
        if ids:
            array = (ctypes.c_longlong * len(ids))(*ids)
            with self._inside() as handle:
                self._check(handle, self.lib.gb_ucx_wait(handle, array, len(ids),
                                                         max(0.0, deadline - time.monotonic())))

    def poll(self, ids: Sequence[int]) -> bool:
        """Progress a little without waiting; True once every operation of ``ids`` is complete."""
        if not ids:
            return True
        array = (ctypes.c_longlong * len(ids))(*ids)
        with self._inside() as handle:
            return self._check(handle, self.lib.gb_ucx_poll(handle, array, len(ids))) == 0

    # -- the interface of a tagged bridge's worker
    def all_reduce(self, pointer: int, count: int, dtype: int, op: int, chunk_elems: int, number: int,
                   deadline: float) -> None:
        with self._inside() as handle:
            self._check(handle, self.lib.gb_ucx_all_reduce(handle, pointer, count, dtype, op, chunk_elems, number,
                                                           max(0.0, deadline - time.monotonic())))

    def broadcast(self, pointer: int, nbytes: int, root: int, chunk_bytes: int, number: int,
                  deadline: float) -> None:
        with self._inside() as handle:
            self._check(handle, self.lib.gb_ucx_broadcast(handle, pointer, nbytes, root, chunk_bytes, number,
                                                          max(0.0, deadline - time.monotonic())))

    def abort(self) -> None:
        try:
            with self._inside() as handle:
                self.lib.gb_ucx_abort(handle)
        except UcxError:
            pass                                           # closed already

    def invalidate(self, pointer: int, nbytes: int) -> None:
        """UCX keeps its own registration cache; a staging buffer needs no word from us."""

    def telemetry(self) -> dict:
        seven = (ctypes.c_ulonglong * 7)()
        with self._inside() as handle:
            self.lib.gb_ucx_counters(handle, seven)
        names = ("sends", "receives", "bytes_out", "bytes_in", "progress_calls", "open_operations", "broken")
        return dict(zip(names, (int(v) for v in seven)))

    def close(self, limit: float = 10.0) -> None:
        def free(handle: int) -> None:
            if self.lib.gb_ucx_close(handle, limit) != 0:
                log.warning("gpubridge_b200: UCX endpoints were still flushing after %g s; the worker was "
                            "torn down anyway", limit)
        self._retire(self.lib.gb_ucx_abort, free)
