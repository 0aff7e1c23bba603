"""Switch memory of a team: NVLink multicast objects made by the fabric itself.

For the in-switch all-reduce (``csrc/gb_switch.cu``) every rank needs memory that is bound to
a multicast object shared with the other members of its group, mapped twice: at a local
address and at the group's multicast address.  This module builds that, once per team, from
the driver's virtual-memory calls (``csrc/gb_mcast.cu``): one member creates the object, the
handle travels to the others as a file descriptor over a Unix socket, every member adds its
GPU, and only then binds its own memory (all devices must have joined before the first bind).

Two kinds of group per team: the whole team (one island, or the flat mode of several), and -
when the team has several islands - this rank's island, for the hierarchical order (island
sums in the switch, the islands' sums exchanged over peer memory).  The reference has no
counterpart: its islands reduce with NCCL/RCCL calls and meet on the host
(src/gpubridge/policies.py:342-357).

A rank that exits while its memory is bound to a multicast object can raise NVLink errors on
the other members' GPUs, so tests that let a rank leave run with ``GPUBRIDGE_NVLS=0``.
"""
from __future__ import annotations

import ctypes
import dataclasses
import os
import socket
import uuid
from datetime import timedelta

from gpubridge_b200.ops import _lib

MIB = 1 << 20
DEFAULT_BYTES = 256 * MIB
FLAG_AREA = _lib.SWITCH_MAX_BLOCKS * _lib.MAX_RANKS * 4           # one row of flags per block index


class SwitchUnavailable(RuntimeError):
    """This machine, driver or team cannot bind multicast memory; the caller falls back."""


@dataclasses.dataclass
class Group:
    """One multicast group as this rank holds it."""
    members: list[int]                 # team indices, in group order
    bytes: int
    object: int = 0                    # the multicast handle
    memory: int = 0                    # this rank's physical allocation
    local: int = 0                     # address of the memory
    multicast: int = 0                 # address of the whole group
    bound: bool = False
    device: int = 0

    def release(self, lib) -> None:
        """Undo every step that succeeded, in reverse.  Never raises."""
        if self.multicast:
            lib.gb_vmm_unmap(self.multicast, self.bytes)
        if self.local:
            lib.gb_vmm_unmap(self.local, self.bytes)
        if self.bound:
            lib.gb_mc_unbind(self.object, self.device, self.bytes)
        if self.memory:
            lib.gb_vmm_release(self.memory)
        if self.object:
            lib.gb_vmm_release(self.object)
        self.multicast = self.local = self.memory = self.object = 0
        self.bound = False


def _check(lib, code: int, what: str) -> None:
    if code != 0:
        raise SwitchUnavailable(f"{what}: {lib.gb_mc_error_string(code).decode()} ({code})")


def _address(token: str, index: int) -> str:
    return f"\0gpubridge-{token}-{index}"          # abstract namespace: nothing to unlink


def exchange_among(store, key: str, me: int, members: list[int], value: str,
                   timeout: timedelta | None) -> list[str]:
    """All-to-all of short strings among ``members`` (team indices) through the store."""
    import time
    store.set(f"{key}/{me}", value)
    keys = [f"{key}/{m}" for m in members]
    deadline = time.monotonic() + (timeout or timedelta(minutes=5)).total_seconds()
    while True:
        try:
            store.wait(keys, timedelta(seconds=max(0.05, min(5.0, deadline - time.monotonic()))))
            break
        except Exception:  # noqa: BLE001 - the store's timeout type differs between stores
            if time.monotonic() >= deadline:
                raise SwitchUnavailable(f"members never reported ({key})") from None
    return [store.get(k).decode() for k in keys]


def _pass_descriptor(store, key: str, me: int, members: list[int], fd: int | None,
                     timeout: timedelta | None) -> int:
    """Hand the creator's (``members[0]``) descriptor to every other member; returns this
    rank's descriptor (its own to close).  The socket names carry a random token, so two jobs
    on one machine never meet."""
    creator = members[0]
    seconds = min(60.0, (timeout or timedelta(minutes=5)).total_seconds())
    if me == creator:
        token = uuid.uuid4().hex
        store.set(f"{key}/token", token)
        for member in members[1:]:
            store.wait([f"{key}/listening/{member}"], timedelta(seconds=seconds))
            with socket.socket(socket.AF_UNIX, socket.SOCK_STREAM) as peer:
                peer.settimeout(seconds)
                peer.connect(_address(token, member))
                socket.send_fds(peer, [b"h"], [fd])
        return fd
    store.wait([f"{key}/token"], timedelta(seconds=seconds))
    token = store.get(f"{key}/token").decode()
    with socket.socket(socket.AF_UNIX, socket.SOCK_STREAM) as listener:
        listener.settimeout(seconds)
        listener.bind(_address(token, me))
        listener.listen(1)
        store.set(f"{key}/listening/{me}", "1")
        connection, _ = listener.accept()
        with connection:
            connection.settimeout(seconds)
            _, fds, _, _ = socket.recv_fds(connection, 16, 1)
    if len(fds) != 1:
        raise SwitchUnavailable("the multicast handle did not arrive")
    return fds[0]


def build_group(lib, store, key: str, me: int, members: list[int], device: int, nbytes: int,
                timeout: timedelta | None) -> Group:
    """Create, join, bind and map one group.  Collective over ``members``.  Every step that
    could fail on one member is followed by an exchange of verdicts among them, so that all
    members give up together."""
    group = Group(list(members), 0, device=device)
    position = members.index(me)

    def agree(step: str, error: Exception | None) -> None:
        if len(members) == 1:
            verdicts = ["ok" if error is None else f"no: {error}"]
        else:
            verdicts = exchange_among(store, f"{key}/{step}", me, members,
                                      "ok" if error is None else f"no: {error}", timeout)
        bad = [v for v in verdicts if v != "ok"]
        if bad:
            group.release(lib)
            raise SwitchUnavailable(bad[0] if error is None else str(error))

    error = None
    try:
        granularity = ctypes.c_size_t()
        _check(lib, lib.gb_mc_granularity(device, len(members), nbytes, ctypes.byref(granularity)),
               "cuMulticastGetGranularity")
        group.bytes = -(-nbytes // granularity.value) * granularity.value
        handle = ctypes.c_ulonglong()
        if position == 0:
            _check(lib, lib.gb_mc_create(len(members), group.bytes, ctypes.byref(handle)),
                   "cuMulticastCreate")
            group.object = handle.value
    except SwitchUnavailable as failure:
        error = failure
    agree("created", error)
    try:
        if len(members) > 1:
            fd = ctypes.c_int(-1)
            if position == 0:
                _check(lib, lib.gb_vmm_export(group.object, ctypes.byref(fd)),
                       "cuMemExportToShareableHandle")
            received = _pass_descriptor(store, key, me, members, fd.value if position == 0 else None,
                                        timeout)
            try:
                if position != 0:
                    _check(lib, lib.gb_vmm_import(received, ctypes.byref(handle)),
                           "cuMemImportFromShareableHandle")
                    group.object = handle.value
            finally:
                os.close(received)
        _check(lib, lib.gb_mc_add_device(group.object, device), "cuMulticastAddDevice")
    except Exception as failure:  # noqa: BLE001 - store, socket or driver: all mean "not here"
        error = failure
    agree("joined", error)                                    # every device is in: binding may start
    try:
        memory = ctypes.c_ulonglong()
        _check(lib, lib.gb_vmm_create(device, group.bytes, ctypes.byref(memory)), "cuMemCreate")
        group.memory = memory.value
        _check(lib, lib.gb_mc_bind(group.object, group.memory, group.bytes), "cuMulticastBindMem")
        group.bound = True
        pointer = ctypes.c_void_p()
        _check(lib, lib.gb_vmm_map(group.memory, group.bytes, granularity.value, device,
                                   ctypes.byref(pointer)), "cuMemMap (local)")
        group.local = pointer.value
        _check(lib, lib.gb_vmm_map(group.object, group.bytes, granularity.value, device,
                                   ctypes.byref(pointer)), "cuMemMap (multicast)")
        group.multicast = pointer.value
        _check(lib, lib.gb_memset_async(group.local, 0, group.bytes, None), "cudaMemsetAsync")
        _check(lib, lib.gb_device_synchronize(), "cudaDeviceSynchronize")
    except SwitchUnavailable as failure:
        error = failure
    agree("bound", error)
    return group


def supported(lib, device: int) -> bool:
    yes = ctypes.c_int(0)
    return lib.gb_mc_supported(device, ctypes.byref(yes)) == 0 and bool(yes.value)


def describe(group: Group, me: int, owners: int, hier: bool, off_flags: int, off_bridge: int,
             len_bridge: int, bseq: int, reserve: int = 0) -> "_lib.GbSwitch":
    """The structure the kernels take.  ``reserve``: bytes at the end of the group's memory that
    the staging kernels must leave alone (the one-step all-reduce's slots live there)."""
    sw = _lib.GbSwitch()
    sw.uc, sw.mc, sw.bytes = group.local, group.multicast, group.bytes - reserve
    sw.off_flags, sw.off_bridge, sw.len_bridge = off_flags, off_bridge, len_bridge
    sw.bseq = bseq
    sw.group_size, sw.group_pos = len(group.members), group.members.index(me)
    sw.owners, sw.hier = owners, int(hier)
    return sw
