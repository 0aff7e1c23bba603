"""The NVLink fabric of one team: symmetric workspaces and the fused collective kernels.

A team is the set of ranks one group's collectives run over (the world, or a subgroup).
Every rank allocates one workspace, exports it, and maps every peer's (CUDA IPC handles
exchanged through the job's store).  The kernels in ``csrc/gb_collectives.cu`` then move
data with plain loads and stores to peer memory from inside the kernel, synchronise with
flags in the workspaces, and reduce, quantise, average and cast in the same launch.  This
replaces the reference's island ``dist.reduce`` + host-staged bridge + island
``dist.broadcast`` (src/gpubridge/policies.py:342-357) and the separate ``div_`` for AVG
(src/gpubridge/collectives.py:103).

All kernels of a team run on one communication stream, in program order, which must be
the same on every rank (the usual rule for collectives).  Calls made on another stream
are ordered with events both ways, so the caller sees current-stream semantics.

Device-side waits are bounded (``GPUBRIDGE_WAIT_TIMEOUT_MS``, default 30 s).  When one
runs out the kernel writes a status record to mapped host memory and returns;
:meth:`Fabric.check` turns it into an exception and poisons the rank, like a failed async
collective.
"""
from __future__ import annotations

import contextlib
import ctypes
import dataclasses
import os
import threading
import time
from datetime import timedelta

import torch

from gpubridge_b200._mutation import mutated

from gpubridge_b200 import config as _config
from gpubridge_b200 import observe as _observe
from gpubridge_b200 import work as _work
from gpubridge_b200.ops import _lib

MIB = 1 << 20
FLAG_BYTES = 4096
ONESHOT_MAX = 1 << 20
NVLS_DTYPES = (torch.float32, torch.bfloat16, torch.float16)            # largest tensor the one-shot kernel takes
# Measured with bench/bench_link.py on B200 (2 ranks): one block moves about 45 GB/s of any
# traffic, a link direction saturates near 650-700 GB/s (16 blocks), a team barrier inside a
# kernel costs about 10 us.  The pipeline plan below is sized from these.
BLOCK_GBS, LINK_GBS, BARRIER_S = 45e9, 650e9, 10e-6
DEFAULT_BYTES = 384 * MIB
THREADS = 512


def _align_down(value: int, multiple: int) -> int:
    return value // multiple * multiple


def _align_up(value: int, multiple: int) -> int:
    return -(-value // multiple) * multiple


@dataclasses.dataclass(frozen=True)
class HierPlan:
    channels: int
    grid: int
    stripe: int          # elements per stripe of a chunk (a multiple of 256)
    nchunks: int
    len_a: int           # bytes of one buffer of each region, per channel
    len_b: int
    len_c: int


def plan_hier(n: int, esize: int, *, k: int, m_max: int, n_islands: int, len_ha: int, len_hb: int,
              len_hc: int, grid: int, chunk_bytes: int | None = None,
              force_channels: int | None = None, force_chunks: int | None = None,
              stripe_multiple: int = 256) -> HierPlan:
    """Channels, chunking and buffer sizes of one hierarchical all-reduce.

    Pure arithmetic on values every rank of the team shares (never this rank's own island
    size or position): all ranks must come out with the same plan, or their stripes do not
    line up.  Every channel owns two buffers of each region; a stripe fits the smallest slot
    (``m_max`` slots in region A, ``n_islands`` in region B, one in region C).  ``stripe_multiple``:
    the stripe length is a multiple of it (256 values; 256 * islands for the two-shot bridge,
    whose sub-stripes must be whole quantisation-block multiples too).

    ``grid`` is one of those shared values too, although it comes from the calling thread's
    grid cap (``Fabric.grid_cap``): a collective is one call on every rank, made from the same
    place in the program - inside the same ``grid_cap`` block or on the same async path - so
    the cap is the same everywhere; a program that caps one rank's call and not its peers' is
    as wrong as one that passes them different sizes."""
    nbytes = n * esize
    # Channels: independent pipelines that hide each other's barriers and local phases.
    # One for small tensors (a barrier costs more than the data), up to four for large.
    channels = force_channels or (1 if nbytes < (4 << 20) else 2 if nbytes < (32 << 20) else 4)
    channels = max(1, min(channels, grid // 8 or 1, 8))
    grid = max(channels, grid // channels * channels)
    len_a = len_ha // channels // 4096 * 4096
    len_b = len_hb // channels // 4096 * 4096
    len_c = len_hc // channels // 4096 * 4096
    slot = min(len_a // m_max, len_b // n_islands, len_c)
    stripe_cap = _align_down(slot // esize, stripe_multiple)
    if stripe_cap < stripe_multiple:
        raise RuntimeError("the fabric workspace is too small for this team; raise "
                           f"{_config.FABRIC_BYTES_ENV}")
    if chunk_bytes:
        want = max(256, chunk_bytes // esize // k)
    else:
        # per channel: T(c) = (c + depth) * (barrier + link time / c) is least at
        # c = sqrt(depth * link time / barrier)
        share = max((m_max - 1) / m_max, (n_islands - 1) / k if n_islands > 1 else 0.0)
        depth = 3 if n_islands > 1 else 2
        link_s = nbytes / channels * share / LINK_GBS
        chunks = force_chunks or max(1, round((depth * link_s / BARRIER_S) ** 0.5))
        want = -(-n // (chunks * channels * k))
    stripe = min(stripe_cap, _align_up(max(1, min(want, -(-n // k))), stripe_multiple))
    return HierPlan(channels, grid, stripe, -(-n // (stripe * k)), len_a, len_b, len_c)


def _bounds_checked(method):
    """With the checked library loaded (``GPUBRIDGE_BOUNDS=1``): allow the launch the
    workspaces, switch memory and the call's own tensors, wait for it, and raise if a kernel
    tried to touch anything else.  Otherwise the method as it is."""
    if not _lib.BOUNDS:
        return method

    import functools

    @functools.wraps(method)
    def run(self, *args, **kwargs):
        tensors = [a for a in (*args, *kwargs.values()) if isinstance(a, torch.Tensor)]
        self._bounds_allow(tensors)
        try:
            return method(self, *args, **kwargs)
        finally:
            self._bounds_verdict(method.__name__)
    return run


class FabricError(RuntimeError):
    """A device-side wait of a fused collective ran out, or the team was poisoned."""


class Fabric:
    """One rank's side of a team.  Build with :func:`create`."""

    def __init__(self, lib, layout, rank: int, device: torch.device, ws: list[int],
                 ws_bytes: int, ctrl: int, status: int, timeout_ms: int, store=None,
                 key: str = "") -> None:
        self.lib, self.layout, self.device = lib, layout, device
        self._store, self._key = store, key
        self.global_rank = rank
        self.rank = layout.index(rank)
        self.world = layout.world_size
        self.ws, self.ws_bytes, self.ctrl, self.status = ws, ws_bytes, ctrl, status
        self.comm_stream = torch.cuda.Stream(device, priority=-1)
        self.max_blocks = int(os.environ.get("GPUBRIDGE_FABRIC_BLOCKS", "128"))
        self._caps = threading.local()          # per-thread grid cap, see grid_cap()
        self.algo = _config.algo_setting()
        self._status = (ctypes.c_uint * _lib.STATUS_WORDS).from_address(status)
        self._residuals: dict[tuple, tuple[torch.Tensor, tuple]] = {}
        self._lock = threading.Lock()
        self._closed = False
        self._role_cache: dict[int, tuple[int, int]] = {}
        # tuning overrides (benchmarks): fixed pipeline depth and role split
        self.force_chunks = int(os.environ.get("GPUBRIDGE_HIER_CHUNKS", "0")) or None
        self.force_channels = int(os.environ.get("GPUBRIDGE_HIER_CHANNELS", "0")) or None
        # Grids of the copy-shaped collectives.  With the bulk-copy ring 16 CTAs already run a
        # link at 640-680 GB/s (measured), so all-gather and broadcast take few SMs and leave
        # the rest to the compute they overlap with; reduce-scatter also reduces locally.
        self.two_shot = os.environ.get("GPUBRIDGE_BRIDGE_TWO_SHOT", "0") == "1"
        self.nvls = None        # (tensor, handle, local pointer, multicast pointer, bytes per buffer)
        # switch memory bound by the fabric itself (enable_switch): the team's group, this
        # rank's island's group, and the structures the kernels take
        self._switch_groups: list = []
        self._heaps: list = []          # (first address, bytes, GbSwitch) of tensors handed out by switch_empty
        self.switch_error = ""          # why enable_switch() said no, for reports
        self.sw_team = self.sw_island = None
        self._bseq = 0
        self.switch_min_bytes = _config.size_setting("GPUBRIDGE_SWITCH_MIN_BYTES", 64 << 10, multiple=1)
        # One NVSwitch joins every GPU of the team, so an uncompressed sum over several islands is
        # reduced in the switch across the whole team (one step, about (n + 1) / n of the tensor
        # per GPU); "0" keeps the hierarchical order in the switch (a group per island, the
        # islands' sums exchanged over peer memory), which moves more and is about half as fast.
        self.switch_flat = os.environ.get("GPUBRIDGE_SWITCH_FLAT", "1") == "1"
        # Through the switch a GPU moves (n + 1) / n of the tensor, over peer memory 2 (n - 1) / n:
        # less from four ranks on, more at two (measured at two: the peer-memory kernels win).
        self.switch_min_ranks = int(os.environ.get("GPUBRIDGE_SWITCH_MIN_RANKS", "3"))
        # The one-step form (copy in, one barrier, every rank reduces the whole tensor in the
        # switch) for tensors up to this size: n times the two-step form's traffic, one barrier
        # and two copies less.  16 MiB / world, at most 4 MiB; 0 turns it off.
        self.switch_oneshot_max = _config.size_setting(
            "GPUBRIDGE_SWITCH_ONESHOT_MAX_BYTES", max(1, min(4 << 20, (16 << 20) // max(1, layout.world_size))),
            multiple=1)
        # A broadcast takes the switch from this many bytes on (measured on four B200s: 548 us
        # against 795 us at 256 MiB, the same at 32 MiB).  Reduce-scatter and all-gather through
        # the switch ran no faster than the peer-memory kernels there (483 against 467 us, 472
        # against 422 us at 256 MiB), so they take it only when asked to
        # (GPUBRIDGE_SWITCH_GATHER_MIN_BYTES; the sizes are the whole tensor: input of a
        # reduce-scatter, output of an all-gather).
        self.switch_copy_min_bytes = _config.size_setting("GPUBRIDGE_SWITCH_COPY_MIN_BYTES", 32 << 20,
                                                          multiple=1)
        self.switch_gather_min_bytes = _config.size_setting("GPUBRIDGE_SWITCH_GATHER_MIN_BYTES", 1 << 62,
                                                            multiple=1)
        self.nvls_reducers = int(os.environ.get("GPUBRIDGE_NVLS_REDUCERS", "48"))
        # 32 / 64 CTAs: stand-alone, 128 would be 10-20 % faster at 256 MiB, but FSDP2 issues these
        # beside its compute and lost 12 % of its step time with 128 (137.9 against 122.3 ms)
        self.copy_blocks = int(os.environ.get("GPUBRIDGE_COPY_BLOCKS", "32"))
        self.overlap_blocks = int(os.environ.get("GPUBRIDGE_OVERLAP_BLOCKS", "32"))
        self.scatter_blocks = int(os.environ.get("GPUBRIDGE_SCATTER_BLOCKS", "64"))
        # reads through the bulk-copy ring (TMA into shared memory) instead of register loads
        # ("phased": one ring run per step instead of one queue per iteration)
        ring = os.environ.get("GPUBRIDGE_RING", "phased")
        self.ring = False if ring == "0" else "phased" if ring == "phased" else True
        self.launches = 0            # kernels launched by this team (benchmarks report it)
        self._engine = None

        islands = layout.islands
        self.n_islands = len(islands)
        self.k = min(len(i.ranks) for i in islands)
        self.m_max = max(len(i.ranks) for i in islands)
        team = _lib.GbTeam()
        team.rank, team.world, team.n_islands = self.rank, self.world, self.n_islands
        team.my_island = layout.island_index(rank)
        team.my_pos = islands[team.my_island].ranks.index(rank)
        position = 0
        for g, island in enumerate(islands):
            team.island_off[g] = position
            for member in island.ranks:
                team.order[position] = layout.index(member)
                position += 1
        team.island_off[self.n_islands] = position
        for r in range(self.world):
            team.ws[r] = ws[r]
        team.ctrl, team.status = ctrl, status
        team.timeout_ns = timeout_ms * 1_000_000
        team.ld_mode = int(os.environ.get("GPUBRIDGE_LD_MODE", "1"))
        self.team = team
        self.my_pos = team.my_pos
        self._plan_regions()

    # -- workspace layout ------------------------------------------------------------------------
    def _plan_regions(self) -> None:
        """Carve the workspace.  Every offset and buffer length is a multiple of 4096."""
        budget = self.ws_bytes - FLAG_BYTES
        cursor = FLAG_BYTES
        # one-shot: [2][world] slots
        # One-shot moves (world - 1) bytes per byte against the pipelined kernel's
        # 2 (world - 1) / world, but needs one barrier instead of three or more: it wins up to
        # about 16 MiB / world (measured crossovers: 4-8 MiB at 2 GPUs, 1-2 MiB at 8).
        self.oneshot_slot = max(ONESHOT_MAX, min(8 * ONESHOT_MAX, 16 * ONESHOT_MAX // max(1, self.world)))
        self.off_oneshot, self.len_oneshot = cursor, self.world * self.oneshot_slot
        cursor += 2 * self.len_oneshot
        # in-switch all-reduce: one flag row per block index, and - several islands - the slots
        # the islands' sums of a stripe are exchanged through
        self.off_swflags = cursor
        cursor += _align_up(_lib.SWITCH_MAX_BLOCKS * _lib.MAX_RANKS * 4, 4096)
        self.off_swbridge = cursor
        self.len_swbridge = (_config.size_setting("GPUBRIDGE_SWITCH_BRIDGE_BYTES", 16 * MIB, multiple=4096)
                             if self.n_islands > 1 else 0)
        cursor += self.len_swbridge
        rest = self.ws_bytes - cursor
        if rest < 16 * MIB:
            raise RuntimeError(f"{_config.FABRIC_BYTES_ENV}: the fabric workspace of "
                               f"{self.ws_bytes} bytes is too small for {self.world} ranks")
        # hierarchical all-reduce gets 45 %, reduce-scatter 30 %, all-gather 20 %, broadcast 5 %
        unit = 4096
        hier = rest * 45 // 100
        per_stripe = hier // (2 * (self.m_max + self.n_islands + 1))
        # one stripe buffer must also hold the largest coded payload (never larger than raw)
        self.stripe_bytes = _align_down(per_stripe, 256 * 8)      # whole blocks of any dtype
        self.off_ha, self.len_ha = cursor, self.m_max * self.stripe_bytes
        cursor += 2 * self.len_ha
        self.off_hb, self.len_hb = cursor, self.n_islands * self.stripe_bytes
        cursor += 2 * self.len_hb
        self.off_hc, self.len_hc = cursor, self.stripe_bytes
        cursor += 2 * self.len_hc
        rs = rest * 30 // 100
        self.rs_chunk_bytes = _align_down(rs // (4 * self.world), unit)
        self.off_rs, self.len_rs = cursor, self.world * self.rs_chunk_bytes
        cursor += 4 * self.len_rs
        ag = rest * 20 // 100
        self.ag_chunk_bytes = _align_down(ag // 4, unit)
        self.off_ag, self.len_ag = cursor, self.ag_chunk_bytes
        cursor += 4 * self.len_ag
        bc = rest * 5 // 100
        self.bc_stripe_bytes = _align_down(bc // 4, unit)
        self.off_bc, self.len_bc = cursor, self.bc_stripe_bytes
        cursor += 4 * self.len_bc
        assert cursor <= self.ws_bytes, (cursor, self.ws_bytes)

    # -- stream discipline --------------------------------------------------------------------------
    def _begin(self):
        current = torch.cuda.current_stream(self.device)
        if current != self.comm_stream and not mutated("comm-ignores-caller"):
            self.comm_stream.wait_stream(current)
        return current

    def _end(self, current) -> None:
        if current != self.comm_stream and not mutated("caller-ignores-comm"):
            current.wait_stream(self.comm_stream)

    def on_comm_stream(self, run, tensors) -> torch.cuda.Event:
        """Run ``run()`` with the communication stream current (ordered after the caller's
        stream); returns the event recorded after it.  The async path of the collectives."""
        current = torch.cuda.current_stream(self.device)
        if not mutated("async-ignores-caller"):
            self.comm_stream.wait_stream(current)
        for t in tensors:
            t.record_stream(self.comm_stream)
        # an asynchronous collective runs beside the caller's compute: it takes few SMs
        with self.grid_cap(self.overlap_blocks), torch.cuda.stream(self.comm_stream):
            run()
            done = torch.cuda.Event()
            done.record(self.comm_stream)
        return done

    # -- in-switch reduction ------------------------------------------------------------------------
    def enable_nvls(self, group, nbytes: int | None = None) -> bool:
        """Bind a buffer of this rank to an NVLink multicast object shared with every member of
        ``group`` (a torch process group with exactly this team's ranks), so that large SUM
        all-reduces of one island run through the switch.  Collective over the group.  The
        allocation and the multicast binding are torch's symmetric memory; the kernel is
        ``allreduce_nvls_kernel``.  Returns False - on every rank alike - when the fabric or
        the torch build cannot do it."""
        if self.n_islands != 1 or self.world < 2:
            return False
        try:
            import torch.distributed._symmetric_memory as symm
            nbytes = nbytes or _config.size_setting("GPUBRIDGE_NVLS_BYTES", 192 * MIB, multiple=4096)
            buffer = symm.empty(nbytes, dtype=torch.uint8, device=self.device)
            handle = symm.rendezvous(buffer, group)
            multicast = int(getattr(handle, "multicast_ptr", 0) or 0)
        except Exception:  # noqa: BLE001 - an optional path: any refusal means "not available"
            return False
        if multicast == 0:
            return False
        third = _align_down(nbytes // 3, 16 * self.world * 256)
        self.nvls = (buffer, handle, buffer.data_ptr(), multicast, third)
        return True

    def enable_switch(self, nbytes: int | None = None, timeout: timedelta | None = None) -> bool:
        """Bind memory of every rank to NVLink multicast objects made by the fabric itself - one
        for the team and, with several islands, one per island - so that SUM / AVG all-reduces
        of floats run through the switch (``csrc/gb_switch.cu``).  Collective over the team.
        Returns False - on every rank alike - when the GPUs, the driver or the team cannot."""
        from gpubridge_b200.ops import switch as _switch
        if self._closed or self.sw_team is not None:
            return self.sw_team is not None
        lib, me, device = self.lib, self.rank, self.device.index
        members = list(range(self.world))
        nbytes = nbytes or _config.size_setting("GPUBRIDGE_SWITCH_BYTES", _switch.DEFAULT_BYTES,
                                                multiple=4096)
        key = f"{self._key}/switch"
        torch.cuda.set_device(self.device)

        def everyone(step: str, ok: bool) -> bool:
            if self.world == 1:
                return ok
            return all(v == "1" for v in _switch.exchange_among(
                self._store, f"{key}/{step}", me, members, "1" if ok else "0", timeout))

        try:
            if not everyone("supported", _switch.supported(lib, device)):
                self.switch_error = "a GPU of the team cannot join a multicast object (no NVSwitch multicast)"
                return False
            groups = []
            try:
                team_group = _switch.build_group(lib, self._store, f"{key}/team", me, members, device,
                                                 nbytes, timeout)
                groups.append(team_group)
                built = True
            except _switch.SwitchUnavailable as failure:
                built = False
                self.switch_error = str(failure)
            if not everyone("team", built):
                for g in groups:
                    g.release(lib)
                return False
            island_group = None
            if self.n_islands > 1 and not self.switch_flat:
                island = self.layout.islands[self.team.my_island]
                mine = [self.layout.index(r) for r in island.ranks]
                try:
                    island_group = _switch.build_group(
                        lib, self._store, f"{key}/island{self.team.my_island}", me, mine, device,
                        nbytes, timeout)
                except _switch.SwitchUnavailable as failure:
                    island_group = None
                    self.switch_error = f"island group: {failure}"
                if not everyone("islands", island_group is not None):
                    if island_group is not None:
                        island_group.release(lib)
                    island_group = None
                else:
                    groups.append(island_group)
        except _switch.SwitchUnavailable as failure:
            self.switch_error = str(failure)
            return False
        bseq = ctypes.c_void_p()
        _lib.check(lib.gb_symm_alloc(4096, ctypes.byref(bseq)), "cudaMalloc (switch barrier numbers)")
        self._bseq = bseq.value
        self._switch_groups = groups
        # the one-step all-reduce's slots sit behind what the staging kernels may use
        reserve = _lib.SWITCH_ONESHOT_RESERVE if team_group.bytes >= 4 * _lib.SWITCH_ONESHOT_RESERVE else 0
        if not reserve:
            self.switch_oneshot_max = 0
        self.sw_team = _switch.describe(team_group, me, self.world, False, self.off_swflags, 0, 0,
                                        self._bseq, reserve)
        if island_group is not None:
            self.sw_island = _switch.describe(island_group, me, self.k, True, self.off_swflags,
                                              self.off_swbridge, self.len_swbridge, self._bseq)
        # Commissioning: one small all-reduce with a known answer through every group, with a
        # short wait limit.  A group that answers wrongly or not at all is given up by every
        # rank alike, and the team stays on the peer-memory kernels.
        if self.world > 1:
            flat_ok = everyone("check-team", self._commission(self.sw_team))
            hier_ok = self.sw_island is None or everyone("check-islands", self._commission(self.sw_island))
            if not hier_ok:
                self.switch_error = "the island groups failed their first sum; using the team's group"
                self.sw_island = None
                # the failed kernel left the per-block barrier numbers out of step: start them over
                self.lib.gb_memset_async(self._bseq, 0, 4096, None)
                self.lib.gb_memset_async(self.ws[self.rank] + self.off_swflags, 0,
                                         _lib.SWITCH_MAX_BLOCKS * _lib.MAX_RANKS * 4, None)
                self.lib.gb_device_synchronize()
                everyone("flags-reset", True)
            if not flat_ok:
                self.switch_error = "the team's group failed its first sum; in-switch reduction is off"
                self._release_switch()
                return False
            if self.switch_oneshot_max and not everyone("check-one-step", self._commission(self.sw_team, True)):
                self.switch_error = "the one-step all-reduce failed its first sum; it stays off"
                self.switch_oneshot_max = 0
                self.lib.gb_memset_async(self._bseq, 0, 4096, None)
                self.lib.gb_memset_async(self.ws[self.rank] + self.off_swflags, 0,
                                         _lib.SWITCH_MAX_BLOCKS * _lib.MAX_RANKS * 4, None)
                self.lib.gb_device_synchronize()
                everyone("flags-reset-2", True)
        if self._engine:
            self._engine_switch()
        return True

    def _commission(self, switch, one_step: bool = False) -> bool:
        """One all-reduce of 96 Ki integer-valued floats through ``switch`` (``one_step``: by the
        one-step kernel); True when this rank got the exact sum in time.  Never raises; clears
        a timeout it caused."""
        n, world = 96 << 10, self.world
        ramp = (torch.arange(n, device=self.device) % 13).float()
        mine, out = ramp + self.rank, torch.full((n,), -1.0, device=self.device)
        want = ramp * world + world * (world - 1) / 2
        saved = self.team.timeout_ns
        self.team.timeout_ns = 3_000_000_000
        try:
            with torch.cuda.stream(self.comm_stream):
                self.comm_stream.wait_stream(torch.cuda.current_stream(self.device))
                entry = self.lib.gb_switch_all_reduce_oneshot if one_step else self.lib.gb_switch_all_reduce
                code = entry(ctypes.byref(self.team), ctypes.byref(switch), mine.data_ptr(),
                             out.data_ptr(), n, 0, 0, 16, self.comm_stream.cuda_stream)
            self.comm_stream.synchronize()
            good = code == 0 and self._status[0] == 0 and bool(torch.equal(out, want))
        except Exception:  # noqa: BLE001 - any failure means "not this way"
            good = False
        finally:
            self.team.timeout_ns = saved
        if self._status[0] != 0:                     # a wait ran out: forget it, the group is dropped
            for word in range(_lib.STATUS_WORDS):
                self._status[word] = 0
            self.lib.gb_memset_async(self.ctrl + 16, 0, 4, None)
            self.lib.gb_device_synchronize()
        return good

    def switch_empty(self, numel: int, dtype: torch.dtype = torch.float32,
                     timeout: timedelta | None = None) -> torch.Tensor | None:
        """A zeroed tensor that lives in switch memory of its own - bound to a multicast object
        of the whole team, at the same offset on every rank - so that all-reduces of it (or of
        16-byte aligned slices of it) run IN PLACE in the switch, with no staging copies: what
        a trainer wants for its gradient buffer.  Collective over the team: every rank calls
        it with the same size.  None - on every rank alike - when the team has no switch
        memory (``enable_switch`` said no, or ``GPUBRIDGE_NVLS=0``).  The memory lives until the
        fabric closes."""
        from gpubridge_b200.ops import switch as _switch
        if self.sw_team is None or self._closed:
            return None
        esize = torch.empty(0, dtype=dtype).element_size()
        nbytes = max(_align_up(numel * esize, 4096), 2 * MIB)
        try:
            group = _switch.build_group(self.lib, self._store, f"{self._key}/switch/heap{len(self._heaps)}",
                                        self.rank, list(range(self.world)), self.device.index, nbytes,
                                        timeout)
        except _switch.SwitchUnavailable as failure:
            self.switch_error = f"switch_empty: {failure}"
            return None
        self._switch_groups.append(group)
        sw = _switch.describe(group, self.rank, self.world, False, self.off_swflags, 0, 0, self._bseq)
        whole = torch.as_tensor(_Foreign(group.local, group.bytes), device=self.device)
        # commissioning, as for the staged groups: a known sum in place, then zeros again
        n, world = min(96 << 10, group.bytes // 4), self.world
        probe = whole[:4 * n].view(torch.float32)
        ramp = (torch.arange(n, device=self.device) % 13).float()
        probe.copy_(ramp + self.rank)
        saved, self.team.timeout_ns = self.team.timeout_ns, 3_000_000_000
        with torch.cuda.stream(self.comm_stream):
            self.comm_stream.wait_stream(torch.cuda.current_stream(self.device))
            code = self.lib.gb_switch_all_reduce_inplace(ctypes.byref(self.team), ctypes.byref(sw), 0, n, 0, 0,
                                                         16, self.comm_stream.cuda_stream)
        self.comm_stream.synchronize()
        self.team.timeout_ns = saved
        good = code == 0 and self._status[0] == 0 and bool(
            torch.equal(probe, ramp * world + world * (world - 1) / 2))
        verdicts = _switch.exchange_among(self._store, f"{self._key}/switch/heap{len(self._heaps)}/check",
                                          self.rank, list(range(self.world)), "1" if good else "0", timeout)
        probe.zero_()
        torch.cuda.synchronize(self.device)
        if "0" in verdicts:
            self.switch_error = "switch_empty: the first in-place sum failed"
            if self._status[0] != 0:
                for word in range(_lib.STATUS_WORDS):
                    self._status[word] = 0
                self.lib.gb_memset_async(self.ctrl + 16, 0, 4, None)
                self.lib.gb_device_synchronize()
            return None
        self._heaps.append((group.local, group.bytes, sw))
        return whole[:numel * esize].view(dtype)

    def _heap_of(self, tensor: torch.Tensor):
        """``(switch, offset)`` when ``tensor`` lies in memory handed out by :meth:`switch_empty`
        and can be reduced in place there, else None."""
        address, nbytes = tensor.data_ptr(), tensor.nbytes
        for first, size, sw in self._heaps:
            if first <= address and address + nbytes <= first + size:
                offset = address - first
                return (sw, offset) if offset % 16 == 0 and nbytes % 16 == 0 else None
        return None

    def _engine_switch(self) -> None:
        self.lib.gb_engine_set_switch(
            self._engine, ctypes.byref(self.sw_team) if self.sw_team is not None else None,
            ctypes.byref(self.sw_island) if self.sw_island is not None else None,
            self.switch_min_bytes, self.switch_min_ranks)
        if self.sw_team is not None:
            self.lib.gb_engine_set_switch_copy(self._engine, self.switch_copy_min_bytes,
                                               self.switch_gather_min_bytes)
            self.lib.gb_engine_set_switch_oneshot(self._engine, self.switch_oneshot_max)

    def _switch_for(self, tensor: torch.Tensor, op: str, compression) -> "_lib.GbSwitch | None":
        """The switch group an all-reduce of ``tensor`` takes, or None for the peer-memory kernels."""
        if (self.sw_team is None or op != "sum" or compression is not None
                or tensor.dtype not in NVLS_DTYPES or tensor.nbytes < self.switch_min_bytes
                or self.world < self.switch_min_ranks):
            return None
        return self.sw_island if self.sw_island is not None else self.sw_team

    def _switch_copy(self, total_bytes: int, *pointers: int, piece: int,
                     gather: bool = True) -> "_lib.GbSwitch | None":
        """The team's switch group when a copy-shaped collective of ``total_bytes`` should take
        it (pieces and pointers in multiples of 16 bytes), else None.  ``gather``: a
        reduce-scatter or all-gather (their own threshold) rather than a broadcast."""
        least = self.switch_gather_min_bytes if gather else self.switch_copy_min_bytes
        if (self.sw_team is None or self.world < self.switch_min_ranks or self.algo != "auto"
                or total_bytes < least or piece % 16
                or any(p % 16 for p in pointers)):
            return None
        return self.sw_team

    def _one_step(self, switch, nbytes: int) -> bool:
        """Whether an all-reduce of ``nbytes`` through ``switch`` takes the one-step kernel: the
        flat group only, small enough, and inside the slots the calling thread's grid has."""
        limit = min(self.max_blocks, getattr(self._caps, "value", 1 << 30))
        blocks = min(2 * limit, _lib.SWITCH_ONESHOT_BLOCKS)
        return (not switch.hier and nbytes <= self.switch_oneshot_max
                and nbytes <= blocks * _lib.SWITCH_ONESHOT_SLOT)

    def _launch_switch_copy(self, call, what: str) -> None:
        limit = min(self.max_blocks, getattr(self._caps, "value", 1 << 30))
        _lib.check(call(limit, torch.cuda.current_stream(self.device).cuda_stream), what)
        self.launches += 1

    # -- the native engine -----------------------------------------------------------------------------
    def engine_config(self) -> "_lib.GbEngineConfig":
        c = _lib.GbEngineConfig()
        c.ws_bytes, c.k, c.m_max = self.ws_bytes, self.k, self.m_max
        c.max_blocks, c.copy_blocks = self.max_blocks, self.copy_blocks
        c.scatter_blocks, c.overlap_blocks = self.scatter_blocks, self.overlap_blocks
        c.ring = 0 if not self.ring else 2 if self.ring == "phased" else 1
        c.two_shot = int(self.two_shot)
        c.force_chunks, c.force_channels = self.force_chunks or 0, self.force_channels or 0
        c.algo = {"auto": 0, "one-shot": 1}.get(self.algo, 2)
        for name in ("oneshot_slot", "off_oneshot", "len_oneshot", "off_ha", "len_ha", "off_hb",
                     "len_hb", "off_hc", "len_hc", "off_rs", "len_rs", "rs_chunk_bytes", "off_ag",
                     "len_ag", "ag_chunk_bytes", "off_bc", "len_bc", "bc_stripe_bytes"):
            setattr(c, name, getattr(self, name))
        return c

    def engine(self) -> int:
        """Handle of this team's native engine (planner and launches in C++, for the C++
        front end), created on first use.  0 when a feature only the Python path has is on
        (in-switch reduction)."""
        if self.nvls is not None or self._closed:
            return 0
        if self._engine is None:
            self._engine = self.lib.gb_engine_create(ctypes.byref(self.team),
                                                     ctypes.byref(self.engine_config()))
            if self._engine and self.sw_team is not None:
                self._engine_switch()
        return self._engine or 0

    # -- health --------------------------------------------------------------------------------------
    def check(self) -> None:
        code = self._status[0]
        if code == 0:
            return
        kinds = {1: "a peer never arrived at a barrier", 2: "a block of the local grid never "
                 "arrived at a barrier", 3: "a bulk copy never landed",
                 4: "a wait inside a tensor-core pipeline ran out"}
        error = FabricError(
            f"gpubridge fused collective failed on team rank {self._status[4]}: "
            f"{kinds.get(code, f'status {code}')} (peer {self._status[1]}, barrier "
            f"{self._status[2]}, step {self._status[3]}) within the device-side wait limit "
            f"({_config.WAIT_MS_ENV})")
        _work.poison(error)
        raise error

    def supports(self, tensors, op: str = "sum") -> bool:
        if self._closed or op not in _lib.OPS:
            return False
        return all(t.device == self.device and t.dtype in _lib.DTYPES and t.is_contiguous()
                   for t in tensors)

    # -- launches --------------------------------------------------------------------------------------
    def _grid(self, nbytes: int, cap: int | None = None) -> int:
        blocks = -(-nbytes // (THREADS * 16 * 4))
        limit = min(cap or self.max_blocks, self.max_blocks, getattr(self._caps, "value", 1 << 30))
        return max(1, min(limit, blocks))

    @contextlib.contextmanager
    def grid_cap(self, blocks: int | None):
        """Launches of the calling thread inside the block use at most ``blocks`` CTAs (a
        collective that runs beside compute should leave it the SMs)."""
        before = getattr(self._caps, "value", 1 << 30)
        self._caps.value = min(before, blocks) if blocks else before
        try:
            yield
        finally:
            self._caps.value = before

    def _launch_reduce(self, kind: int, tensor_dtype, op: str, codec: int, args, grid: int) -> None:
        stream = torch.cuda.current_stream(self.device).cuda_stream
        code = self.lib.gb_launch_reduce(kind, _lib.DTYPES[tensor_dtype], _lib.OPS[op], codec,
                                         ctypes.byref(self.team), ctypes.byref(args), grid, stream)
        _lib.check(code, "gb_launch_reduce")
        self.launches += 1

    def _launch_copy(self, kind: int, args, grid: int) -> None:
        stream = torch.cuda.current_stream(self.device).cuda_stream
        code = self.lib.gb_launch_copy(kind, ctypes.byref(self.team), ctypes.byref(args), grid,
                                       stream)
        _lib.check(code, "gb_launch_copy")
        self.launches += 1

    # -- the checked build ------------------------------------------------------------------------------
    def _bounds_allow(self, tensors) -> None:
        self._bounds_tensors = tensors
        table = _lib.GbBoundsTable()
        ranges = [(int(self.team.ws[r]), int(self.team.ws[r]) + self.ws_bytes) for r in range(self.world)]
        for sw in [self.sw_team, self.sw_island] + [heap[2] for heap in self._heaps]:
            if sw is not None:
                ranges += [(int(sw.uc), int(sw.uc) + sw.bytes), (int(sw.mc), int(sw.mc) + sw.bytes)]
        ranges += [(t.data_ptr(), t.data_ptr() + t.nbytes) for t in tensors if t.numel()]
        for residual in self._residuals.values():
            ranges.append((residual[0].data_ptr(), residual[0].data_ptr() + residual[0].nbytes))
        ranges = ranges[:_lib.BOUNDS_RANGES]
        for i, (lo, hi) in enumerate(ranges):
            table.lo[i], table.hi[i] = lo, hi
        table.n = len(ranges)
        for unit in ("collectives", "switch"):
            _lib.check(getattr(self.lib, f"gb_bounds_set_{unit}")(ctypes.byref(table)), "bounds table")

    def _bounds_verdict(self, what: str) -> None:
        torch.cuda.synchronize(self.device)
        for unit in ("collectives", "switch"):
            table = _lib.GbBoundsTable()
            _lib.check(getattr(self.lib, f"gb_bounds_get_{unit}")(ctypes.byref(table)), "bounds table")
            if table.violations:
                kind = {0: "load", 1: "store", 2: "bulk copy"}.get(int(table.first[1]), "access")
                raise FabricError(
                    f"{what}: {table.violations} accesses outside the allowed memory; the first: a "
                    f"{kind} at {int(table.first[0]):#x} by thread {int(table.first[3])} of block "
                    f"{int(table.first[2])} ({unit} kernels, team rank {self.rank})")

    # -- collectives -----------------------------------------------------------------------------------
    @_bounds_checked
    def all_reduce(self, tensor: torch.Tensor, op: str = "sum", divide: int | None = None,
                   mode: str = "auto", compression=None, chunk_bytes: int | None = None,
                   out: torch.Tensor | None = None, keep: tuple[int, int] | None = None) -> None:
        """Reduce ``tensor`` over the team into ``out`` (default: in place).  ``keep = (first
        element, count)``: only that range of the result is wanted, and ``out`` holds just it (the
        compressed reduce-scatter: the register-load hierarchical kernel, whose last step then
        fetches one slice instead of the whole tensor).

        ``mode``: ``auto`` (one-shot up to 256 KiB, else hierarchical), ``striped``
        (hierarchical always), ``chunked`` (hierarchical, ``chunk_bytes`` per pipeline step).
        ``compression``: ``(mode, format)`` for the cross-island step, SUM of floats only.
        """
        n = tensor.numel()
        if n == 0:
            return
        out = tensor if out is None else out
        nbytes = tensor.nbytes
        if compression is not None and (op != "sum" or self.n_islands < 2):
            compression = None
        algo = self.algo
        oneshot = (compression is None and nbytes <= self.oneshot_slot and keep is None
                   and ((mode == "auto" and algo in ("auto", "one-shot")) or algo == "one-shot"))
        switch = (self._switch_for(tensor, op, compression)
                  if mode == "auto" and algo == "auto" and keep is None else None)
        current = self._begin()
        try:
            with torch.cuda.stream(self.comm_stream):
                args = _lib.GbArgs()
                args.inp, args.out, args.n = tensor.data_ptr(), out.data_ptr(), n
                args.divide = int(divide or 0)
                if keep is not None:
                    args.keep_lo, args.keep_n = keep
                home = None
                if (self._heaps and out is tensor and op == "sum" and compression is None and keep is None
                        and tensor.dtype in NVLS_DTYPES and mode == "auto" and algo == "auto"):
                    home = self._heap_of(tensor)       # in place at any team size: nothing is staged
                if home is not None:
                    limit = min(self.max_blocks, getattr(self._caps, "value", 1 << 30))
                    code = self.lib.gb_switch_all_reduce_inplace(
                        ctypes.byref(self.team), ctypes.byref(home[0]), home[1], n,
                        _lib.DTYPES[tensor.dtype], args.divide, limit,
                        torch.cuda.current_stream(self.device).cuda_stream)
                    _lib.check(code, "gb_switch_all_reduce_inplace")
                    self.launches += 1
                elif switch is not None and self._one_step(switch, nbytes):
                    limit = min(self.max_blocks, getattr(self._caps, "value", 1 << 30))
                    code = self.lib.gb_switch_all_reduce_oneshot(
                        ctypes.byref(self.team), ctypes.byref(switch), args.inp, args.out, n,
                        _lib.DTYPES[tensor.dtype], args.divide, limit,
                        torch.cuda.current_stream(self.device).cuda_stream)
                    _lib.check(code, "gb_switch_all_reduce_oneshot")
                    self.launches += 1
                elif switch is not None:
                    limit = min(self.max_blocks, getattr(self._caps, "value", 1 << 30))
                    code = self.lib.gb_switch_all_reduce(
                        ctypes.byref(self.team), ctypes.byref(switch), args.inp, args.out, n,
                        _lib.DTYPES[tensor.dtype], args.divide, limit,
                        torch.cuda.current_stream(self.device).cuda_stream)
                    _lib.check(code, "gb_switch_all_reduce")
                    self.launches += 1
                    if _observe.watching() and not torch.cuda.is_current_stream_capturing():
                        self._report_switch_phase()
                elif oneshot:
                    args.off_a, args.len_a = self.off_oneshot, self.len_oneshot
                    self._launch_reduce(0, tensor.dtype, op, 0, args, self._grid(nbytes, 32))
                elif (self.nvls is not None and op == "sum" and compression is None
                      and tensor.dtype in NVLS_DTYPES and mode != "chunked"):
                    _, _, local, multicast, third = self.nvls
                    esize = tensor.element_size()
                    args.sym, args.mc = local, multicast
                    args.off_a, args.len_a = 0, third
                    # chunks small enough that the three-stage pipeline fills: at least four
                    chunk = min(third, max(1 << 20, -(-nbytes // 4)))
                    args.chunk = _align_up(chunk, 16 * self.world * 16) // esize
                    if args.chunk * esize > third:
                        args.chunk = _align_down(third, 16 * self.world * 16) // esize
                    grid = self._grid(nbytes)
                    args.k = self.nvls_reducers if grid >= 2 * self.nvls_reducers else 0
                    self._launch_reduce(5, tensor.dtype, op, 0, args, grid)
                else:
                    self._hier(tensor, args, op, compression, chunk_bytes)
        finally:
            self._end(current)

    def _hier(self, tensor, args, op, compression, chunk_bytes) -> None:
        aligned = (args.inp | args.out) % 16 == 0
        ring = bool(self.ring) and compression is None and aligned and not args.keep_n
        # more than two islands: the bridge can move 2 (I - 1) / I stripes per owner instead of
        # I - 1 (GPUBRIDGE_BRIDGE_TWO_SHOT=1; the phased ring kernel only)
        two_shot = (ring and self.ring == "phased" and self.n_islands >= 3 and self.two_shot)
        plan = plan_hier(tensor.numel(), tensor.element_size(), k=self.k, m_max=self.m_max,
                         n_islands=self.n_islands, len_ha=self.len_ha, len_hb=self.len_hb,
                         len_hc=self.len_hc, grid=self._grid(tensor.nbytes * 2),
                         chunk_bytes=chunk_bytes, force_channels=self.force_channels,
                         force_chunks=self.force_chunks,
                         stripe_multiple=256 * self.n_islands if two_shot else 256)
        args.role_b = 1 if two_shot else 0
        args.stripe, args.k, args.chunk = plan.stripe, self.k, plan.stripe * self.k
        args.off_a, args.len_a = self.off_ha, plan.len_a
        args.off_b, args.len_b = self.off_hb, plan.len_b
        args.off_c, args.len_c = self.off_hc, plan.len_c
        args.role_a = plan.channels
        codec = 0
        if compression is not None:
            codec = _lib.CODECS[tuple(compression)]
            args.residual = self._residual(tensor, (plan.stripe, self.k, plan.nchunks, codec)).data_ptr()
        kind = (4 if self.ring == "phased" else 3) if ring else 1
        self._launch_reduce(kind, tensor.dtype, op, codec, args, plan.grid)
        if _observe.watching() and not torch.cuda.is_current_stream_capturing():
            self._report_phases(plan)

    def _report_phases(self, plan: "HierPlan") -> None:
        """Hand observers the kernel's own timestamps: the barriers between the steps of the
        first channel (``globaltimer`` values the kernel leaves in its control block), copied
        to pinned memory behind the kernel - the host does not wait."""
        bridged = self.n_islands > 1
        per_channel = -(-plan.nchunks // plan.channels)
        barriers = min(8, per_channel + (3 if bridged else 2) - 1)
        if barriers < 2:
            return
        if per_channel == 1:
            names = ["island-reduce", "bridge-reduce"][:barriers - 1]
        else:
            names = [f"pipeline-step-{i + 1}" for i in range(barriers - 1)]
        stamps = torch.zeros(8, dtype=torch.int64).pin_memory()
        stream = torch.cuda.current_stream(self.device)
        _lib.check(self.lib.gb_copy_to_host(stamps.data_ptr(), self.ctrl + 32, 64, stream.cuda_stream),
                   "cudaMemcpyAsync (barrier timestamps)")
        done = torch.cuda.Event(enable_timing=True)
        done.record(stream)
        _observe.device_phases_later(names, stamps, done)

    def _report_switch_phase(self) -> None:
        """The in-switch all-reduce as observers see it: one phase, from the moment block 0 has
        met its peers for the first time (every rank's first tiles are staged) to the moment its
        last tile is out - ``globaltimer`` values the kernel leaves, copied behind it."""
        stamps = torch.zeros(8, dtype=torch.int64).pin_memory()
        stream = torch.cuda.current_stream(self.device)
        _lib.check(self.lib.gb_copy_to_host(stamps.data_ptr(), self.ctrl + 32, 64, stream.cuda_stream),
                   "cudaMemcpyAsync (switch timestamps)")
        done = torch.cuda.Event(enable_timing=True)
        done.record(stream)
        _observe.device_phases_later(["switch-reduce"], stamps, done)

    def _residual(self, tensor: torch.Tensor, geometry: tuple) -> torch.Tensor:
        """Error feedback of this rank's stripes of ``tensor``: found by the buffer's address,
        size and dtype (reference: compression.py:321-324); zero the first time or when the
        chunk geometry changed."""
        key = (tensor.data_ptr(), tensor.numel(), tensor.dtype)
        with self._lock:
            kept = self._residuals.get(key)
            if kept is None or kept[1] != geometry:
                stripe, _, nchunks, _ = geometry
                size = stripe * nchunks if self.my_pos < self.k else 256
                kept = (torch.zeros(size, dtype=torch.float32, device=self.device), geometry)
                self._residuals[key] = kept
                if _lib.BOUNDS:
                    self._bounds_allow(getattr(self, "_bounds_tensors", []))
            return kept[0]

    def reset_error_feedback(self) -> None:
        with self._lock:
            self._residuals.clear()

    @_bounds_checked
    def reduce_scatter(self, output: torch.Tensor, tensor: torch.Tensor, divide: int | None = None,
                       compression=None) -> None:
        """``output`` = slice ``rank`` of the sum of every rank's ``tensor``."""
        n = output.numel()
        if n == 0:
            return
        if compression is not None and self.n_islands > 1:
            # compressed bridge leg: the hierarchical all-reduce - island sums, quantised, across
            # the bridge, added in island order - whose last step fetches this rank's slice only,
            # straight into `output`: the same bits as the compressed all-reduce's slice
            self.all_reduce(tensor, "sum", divide, "striped", compression, out=output,
                            keep=(self.rank * n, n))
            return
        esize = tensor.element_size()
        # a float input may leave as bf16 and a bf16 input as float: the cast is the sum's one
        # rounding instead of a pass of its own over the result
        casting = output.dtype != tensor.dtype
        if casting and {output.dtype, tensor.dtype} != {torch.float32, torch.bfloat16}:
            raise ValueError("reduce_scatter casts between float32 and bfloat16 only, got "
                             f"{tensor.dtype} -> {output.dtype}")
        switch = None if casting or tensor.dtype not in NVLS_DTYPES else self._switch_copy(
            tensor.nbytes, tensor.data_ptr(), output.data_ptr(), piece=n * esize)
        current = self._begin()
        try:
            with torch.cuda.stream(self.comm_stream):
                if switch is not None:
                    self._launch_switch_copy(lambda limit, stream: self.lib.gb_switch_reduce_scatter(
                        ctypes.byref(self.team), ctypes.byref(switch), tensor.data_ptr(), output.data_ptr(),
                        n, _lib.DTYPES[tensor.dtype], int(divide or 0), limit, stream),
                        "gb_switch_reduce_scatter")
                    return
                args = _lib.GbArgs()
                args.inp, args.out, args.n = tensor.data_ptr(), output.data_ptr(), n
                args.divide = int(divide or 0)
                args.chunk = min(_align_down(self.rs_chunk_bytes // esize, 256),
                                 _align_up(n, 256))
                args.off_a, args.len_a = self.off_rs, self.len_rs
                grid = self._grid(tensor.nbytes, min(self.scatter_blocks, self.max_blocks))
                if -(-n // args.chunk) >= 4 and grid >= 8:
                    args.role_a = grid * 3 // 4
                self._launch_reduce(6 if casting else 2, tensor.dtype, "sum", 0, args, grid)
        finally:
            self._end(current)

    @_bounds_checked
    def all_gather(self, output: torch.Tensor, tensor: torch.Tensor) -> None:
        nbytes = tensor.nbytes
        if nbytes == 0:
            return
        switch = self._switch_copy(output.nbytes, tensor.data_ptr(), output.data_ptr(), piece=nbytes)
        current = self._begin()
        try:
            with torch.cuda.stream(self.comm_stream):
                if switch is not None:
                    self._launch_switch_copy(lambda limit, stream: self.lib.gb_switch_all_gather(
                        ctypes.byref(self.team), ctypes.byref(switch), tensor.data_ptr(), output.data_ptr(),
                        nbytes, limit, stream), "gb_switch_all_gather")
                    return
                args = _lib.GbArgs()
                args.inp, args.out, args.n = tensor.data_ptr(), output.data_ptr(), nbytes
                args.chunk = min(self.ag_chunk_bytes, _align_up(nbytes, 16))
                args.off_a, args.len_a = self.off_ag, self.len_ag
                self._launch_copy(0, args, self._grid(output.nbytes, min(self.copy_blocks, self.max_blocks)))
        finally:
            self._end(current)

    @_bounds_checked
    def broadcast(self, tensor: torch.Tensor, src: int) -> None:
        """Copy ``tensor`` from global rank ``src`` to every rank of the team."""
        nbytes = tensor.nbytes
        if nbytes == 0:
            return
        switch = self._switch_copy(nbytes, tensor.data_ptr(), piece=nbytes, gather=False)
        current = self._begin()
        try:
            with torch.cuda.stream(self.comm_stream):
                if switch is not None:
                    root = self.layout.index(src)
                    self._launch_switch_copy(lambda limit, stream: self.lib.gb_switch_broadcast(
                        ctypes.byref(self.team), ctypes.byref(switch), tensor.data_ptr(), nbytes, root,
                        limit, stream), "gb_switch_broadcast")
                    return
                args = _lib.GbArgs()
                args.out, args.n = tensor.data_ptr(), nbytes
                args.root = self.layout.index(src)
                stripe = min(self.bc_stripe_bytes, _align_up(-(-nbytes // self.world), 16))
                args.stripe, args.chunk = stripe, stripe * self.world
                args.off_a, args.len_a = self.off_bc, self.len_bc
                self._launch_copy(1, args, self._grid(nbytes * 2, min(self.copy_blocks, self.max_blocks)))
        finally:
            self._end(current)

    def barrier(self) -> None:
        current = self._begin()
        try:
            with torch.cuda.stream(self.comm_stream):
                self._launch_copy(2, _lib.GbArgs(), 1)
        finally:
            self._end(current)

    def probe(self, kind: str, nbytes: int = 0, grid: int = 64, repeat: int = 1) -> None:
        """Enqueue the link probe: ``store`` / ``load`` (to / from the next rank), ``copy``
        (local), their ``ring-`` forms (through the bulk-copy ring), or ``barrier`` (``nbytes``
        barriers).  Time it with events on the
        communication stream."""
        args = _lib.GbArgs()
        args.k = {"store": 0, "load": 1, "copy": 2, "barrier": 3, "mixed": 4, "mixed3": 5,
                  "ring-store": 6, "ring-load": 7, "ring-copy": 8}[kind]
        args.n = nbytes if kind == "barrier" else min(nbytes, self.len_ha, self.len_hb,
                                                      self.len_hc)
        args.divide = repeat
        args.off_a, args.off_b, args.off_c = self.off_ha, self.off_hb + self.len_hb, self.off_hc
        args.len_a = self.len_ha
        current = self._begin()
        try:
            with torch.cuda.stream(self.comm_stream):
                self._launch_copy(3, args, grid)
        finally:
            self._end(current)

    # -- teardown ------------------------------------------------------------------------------------------
    def close(self) -> None:
        """Unmap the peers and free the workspace.  A peer may still be loading from this
        rank's workspace in its last kernel, so the ranks first meet on the store after each
        has synchronised its device, unmap, and meet again before anybody frees.  If a peer
        never shows up (it died) the memory is left to process exit rather than freed under
        a running kernel."""
        if self._closed:
            return
        self._closed = True
        if self._engine:
            self.lib.gb_engine_destroy(self._engine)
            self._engine = None
        try:
            torch.cuda.synchronize(self.device)
        except Exception:  # noqa: BLE001 - teardown never raises
            pass
        self.nvls = None
        short = timedelta(seconds=20)
        if self.world == 1:
            self._release_switch()
            self.lib.gb_symm_free(self.ws[0])
            self.lib.gb_symm_free(self.ctrl)
            self.lib.gb_status_free(self.status)
            return
        try:
            _exchange(self._store, self._key + "/closing", self.rank, self.world, "1", short)
            for r, ptr in enumerate(self.ws):
                if r != self.rank and ptr:
                    self.lib.gb_symm_unmap(ptr)
            _exchange(self._store, self._key + "/unmapped", self.rank, self.world, "1", short)
        except Exception:  # noqa: BLE001 - a peer is gone: leak instead of freeing in use
            return
        self._release_switch()
        self.lib.gb_symm_free(self.ws[self.rank])
        self.lib.gb_symm_free(self.ctrl)
        self.lib.gb_status_free(self.status)
        self._residuals.clear()


class _Foreign:
    """Device memory that torch did not allocate, as ``torch.as_tensor`` takes it."""

    def __init__(self, address: int, nbytes: int) -> None:
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "strides": None,
                                         "data": (address, False), "version": 3}


def _release_switch_of(fabric) -> None:
    fabric._heaps = []
    for group in reversed(fabric._switch_groups):
        group.release(fabric.lib)
    fabric._switch_groups = []
    fabric.sw_team = fabric.sw_island = None
    if fabric._bseq:
        fabric.lib.gb_symm_free(fabric._bseq)
        fabric._bseq = 0


Fabric._release_switch = _release_switch_of


def _exchange(store, key: str, rank_index: int, world: int, value: str,
              timeout: timedelta | None) -> list[str]:
    store.set(f"{key}/{rank_index}", value)
    keys = [f"{key}/{r}" for r in range(world)]
    deadline = time.monotonic() + (timeout or timedelta(minutes=30)).total_seconds()
    while True:
        try:
            store.wait(keys, timedelta(seconds=max(0.05, min(5.0, deadline - time.monotonic()))))
            break
        except Exception:  # noqa: BLE001
            if time.monotonic() >= deadline:
                raise RuntimeError(f"gpubridge fabric setup: peers never reported ({key})") from None
    return [store.get(k).decode() for k in keys]


def create_single(device: torch.device) -> Fabric:
    """A team of one rank: no peers, no handles, the same kernels.  For single-GPU use of the
    fused GEMM and for profiling one rank's side of the collectives."""
    from gpubridge_b200.topology import plan_topology
    lib = _lib.lib()
    torch.cuda.set_device(device)
    ws_bytes = _config.size_setting(_config.FABRIC_BYTES_ENV, DEFAULT_BYTES, multiple=4096)
    local, ctrl, status = ctypes.c_void_p(), ctypes.c_void_p(), ctypes.c_void_p()
    _lib.check(lib.gb_symm_alloc(ws_bytes, ctypes.byref(local)), "cudaMalloc (fabric workspace)")
    _lib.check(lib.gb_symm_alloc(max(4096, 8 * lib.gb_sizeof_ctrl()), ctypes.byref(ctrl)),
               "cudaMalloc (control block)")
    _lib.check(lib.gb_status_alloc(4 * _lib.STATUS_WORDS, ctypes.byref(status)), "cudaHostAlloc")
    return Fabric(lib, plan_topology(["nvidia"]), 0, device, [local.value], ws_bytes, ctrl.value,
                  status.value, _config.wait_timeout_ms(), None, "")


def create(store, name: str, layout, rank: int, device: torch.device,
           timeout: timedelta | None = None) -> Fabric | None:
    """Map the team's workspaces.  Collective over the team's members.  Returns None - on
    every member alike - when the team has one rank or more than 16, or some pair of its
    GPUs cannot address each other's memory."""
    world = layout.world_size
    if world < 2 or world > _lib.MAX_RANKS:
        return None
    lib = _lib.lib()
    me = layout.index(rank)
    key = f"gb/{name}/fabric/{'_'.join(map(str, layout.members))}"
    torch.cuda.set_device(device)
    # 1. can every pair reach each other?  (device index + verdict, agreed by all)
    indices = [int(v) for v in _exchange(store, key + "/dev", me, world, str(device.index), timeout)]
    reachable = True
    for other in indices:
        if other != device.index:
            yes = ctypes.c_int(0)
            _lib.check(lib.gb_can_access_peer(device.index, other, ctypes.byref(yes)),
                       "cudaDeviceCanAccessPeer")
            reachable = reachable and bool(yes.value)
    if len(set(indices)) != world:
        reachable = False            # two members on one GPU: kernels that wait on each other
    verdicts = _exchange(store, key + "/p2p", me, world, "1" if reachable else "0", timeout)
    if "0" in verdicts:
        return None
    # 2. allocate, export, import
    ws_bytes = _config.size_setting(_config.FABRIC_BYTES_ENV, DEFAULT_BYTES, multiple=4096)
    local = ctypes.c_void_p()
    _lib.check(lib.gb_symm_alloc(ws_bytes, ctypes.byref(local)), "cudaMalloc (fabric workspace)")
    handle = ctypes.create_string_buffer(64)
    _lib.check(lib.gb_symm_export(local, handle), "cudaIpcGetMemHandle")
    handles = _exchange(store, key + "/ipc", me, world, handle.raw.hex(), timeout)
    ws: list[int] = []
    for r, text in enumerate(handles):
        if r == me:
            ws.append(local.value)
            continue
        mapped = ctypes.c_void_p()
        _lib.check(lib.gb_symm_import(bytes.fromhex(text), ctypes.byref(mapped)),
                   f"cudaIpcOpenMemHandle (team rank {r})")
        ws.append(mapped.value)
    ctrl = ctypes.c_void_p()
    _lib.check(lib.gb_symm_alloc(max(4096, 8 * lib.gb_sizeof_ctrl()), ctypes.byref(ctrl)),
               "cudaMalloc (control block)")
    status = ctypes.c_void_p()
    _lib.check(lib.gb_status_alloc(4 * _lib.STATUS_WORDS, ctypes.byref(status)), "cudaHostAlloc")
    fabric = Fabric(lib, layout, rank, device, ws, ws_bytes, ctrl.value, status.value,
                    _config.wait_timeout_ms(), store, key)
    # 3. nobody launches before everybody has mapped everything
    _exchange(store, key + "/ready", me, world, "1", timeout)
    return fabric
