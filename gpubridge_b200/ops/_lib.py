"""ctypes binding of the native library.

The library is built in-tree by :mod:`gpubridge_b200.ops._build`.  It is loaded after
``import torch`` so the CUDA runtime torch ships is the one both share; kernels receive
``tensor.data_ptr()`` values and the current stream's ``cudaStream_t``.  On a machine with
a GPU a missing library is an error (it is built on the spot if a compiler is there):
nothing silently falls back to eager PyTorch.
"""
from __future__ import annotations

import ctypes
import os
import threading

import torch  # noqa: F401 - loads libcudart before the library below

from gpubridge_b200.ops import _build

MAX_RANKS = 16
STATUS_WORDS = 8
SWITCH_MAX_BLOCKS = 320
SWITCH_ONESHOT_SLOT, SWITCH_ONESHOT_BLOCKS = 32 << 10, 128
SWITCH_ONESHOT_RESERVE = 2 * SWITCH_ONESHOT_SLOT * SWITCH_ONESHOT_BLOCKS

DTYPES = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2, torch.float64: 3,
          torch.int8: 4, torch.uint8: 5, torch.int32: 6, torch.int64: 7}
OPS = {"sum": 0, "max": 1, "min": 2}
CODECS = {None: 0, ("bf16", "ref"): 1, ("bf16", "b200"): 1, ("fp8", "ref"): 2, ("fp8", "b200"): 3}


class GbTeam(ctypes.Structure):
    _fields_ = [("rank", ctypes.c_int), ("world", ctypes.c_int), ("n_islands", ctypes.c_int),
                ("my_island", ctypes.c_int), ("my_pos", ctypes.c_int),
                ("island_off", ctypes.c_int * (MAX_RANKS + 1)),
                ("order", ctypes.c_int * MAX_RANKS),
                ("ws", ctypes.c_void_p * MAX_RANKS),
                ("ctrl", ctypes.c_void_p), ("status", ctypes.c_void_p),
                ("timeout_ns", ctypes.c_ulonglong), ("ld_mode", ctypes.c_int),
                ("pad", ctypes.c_int)]


class GbArgs(ctypes.Structure):
    _fields_ = [("inp", ctypes.c_void_p), ("out", ctypes.c_void_p), ("n", ctypes.c_size_t),
                ("chunk", ctypes.c_size_t), ("stripe", ctypes.c_size_t), ("k", ctypes.c_int),
                ("divide", ctypes.c_int), ("root", ctypes.c_int), ("role_a", ctypes.c_int),
                ("role_b", ctypes.c_int), ("pad", ctypes.c_int),
                ("off_a", ctypes.c_size_t), ("off_b", ctypes.c_size_t), ("off_c", ctypes.c_size_t),
                ("len_a", ctypes.c_size_t), ("len_b", ctypes.c_size_t), ("len_c", ctypes.c_size_t),
                ("residual", ctypes.c_void_p), ("sym", ctypes.c_void_p), ("mc", ctypes.c_void_p),
                ("keep_lo", ctypes.c_size_t), ("keep_n", ctypes.c_size_t)]


class GbSwitch(ctypes.Structure):
    """One rank's view of the switch memory of its group (csrc/gb_switch.h)."""
    _fields_ = [("uc", ctypes.c_void_p), ("mc", ctypes.c_void_p), ("bytes", ctypes.c_size_t),
                ("off_flags", ctypes.c_size_t), ("off_bridge", ctypes.c_size_t),
                ("len_bridge", ctypes.c_size_t), ("bseq", ctypes.c_void_p),
                ("group_size", ctypes.c_int), ("group_pos", ctypes.c_int),
                ("owners", ctypes.c_int), ("hier", ctypes.c_int)]


class GbSwitchPlan(ctypes.Structure):
    _fields_ = [("tile", ctypes.c_size_t), ("ntiles", ctypes.c_int), ("grid", ctypes.c_int)]


class GbEngineConfig(ctypes.Structure):
    """What the native engine needs of a team: grids, switches and the workspace regions."""
    _fields_ = ([("ws_bytes", ctypes.c_size_t)]
                + [(name, ctypes.c_int) for name in (
                    "k", "m_max", "max_blocks", "copy_blocks", "scatter_blocks", "overlap_blocks",
                    "ring", "two_shot", "force_chunks", "force_channels", "algo")]
                + [(name, ctypes.c_size_t) for name in (
                    "oneshot_slot", "off_oneshot", "len_oneshot", "off_ha", "len_ha", "off_hb",
                    "len_hb", "off_hc", "len_hc", "off_rs", "len_rs", "rs_chunk_bytes", "off_ag",
                    "len_ag", "ag_chunk_bytes", "off_bc", "len_bc", "bc_stripe_bytes")])


BOUNDS = os.environ.get("GPUBRIDGE_BOUNDS", "0") == "1"
"""The checked library (``-DGB_BOUNDS``) is the one loaded: a debugging run."""
BOUNDS_RANGES = 40
BOUNDS_UNITS = ("collectives", "switch", "gemm", "gemm2", "gemm_rs")


class GbBoundsTable(ctypes.Structure):
    _fields_ = [("lo", ctypes.c_ulonglong * BOUNDS_RANGES), ("hi", ctypes.c_ulonglong * BOUNDS_RANGES),
                ("n", ctypes.c_int), ("pad", ctypes.c_int), ("first", ctypes.c_ulonglong * 4),
                ("violations", ctypes.c_uint), ("pad2", ctypes.c_uint)]


def path() -> str:
    return _build.LIB_BOUNDS if BOUNDS else _build.LIB


class GbLaunch(ctypes.Structure):
    _fields_ = [("family", ctypes.c_int), ("kind", ctypes.c_int), ("grid", ctypes.c_int),
                ("args", GbArgs)]


class GbHierPlanOut(ctypes.Structure):
    _fields_ = [("channels", ctypes.c_int), ("grid", ctypes.c_int), ("stripe", ctypes.c_size_t),
                ("nchunks", ctypes.c_size_t), ("len_a", ctypes.c_size_t),
                ("len_b", ctypes.c_size_t), ("len_c", ctypes.c_size_t)]


_lock = threading.Lock()
_lib: ctypes.CDLL | None = None


def available() -> bool:
    return os.path.exists(path())


def lib() -> ctypes.CDLL:
    """The loaded library; builds it first when it is missing and nvcc is there."""
    global _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not os.path.exists(path()):
            _build.build(bounds=BOUNDS)
        loaded = ctypes.CDLL(path())
        _declare(loaded)
        if loaded.gb_sizeof_team() != ctypes.sizeof(GbTeam) or \
                loaded.gb_sizeof_args() != ctypes.sizeof(GbArgs) or \
                loaded.gb_sizeof_engine_config() != ctypes.sizeof(GbEngineConfig) or \
                loaded.gb_sizeof_launch() != ctypes.sizeof(GbLaunch) or \
                loaded.gb_sizeof_switch() != ctypes.sizeof(GbSwitch):
            raise RuntimeError("the native library's structures do not match ops/_lib.py; "
                               "rebuild with python -m gpubridge_b200.ops._build --force")
        _lib = loaded
        return loaded


def _declare(L: ctypes.CDLL) -> None:
    vp, sz, i = ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int
    if BOUNDS:
        for unit in BOUNDS_UNITS:
            for verb in ("set", "get"):
                getattr(L, f"gb_bounds_{verb}_{unit}").argtypes = [ctypes.POINTER(GbBoundsTable)]
    L.gb_error_string.restype = ctypes.c_char_p
    L.gb_error_string.argtypes = [i]
    for name in ("gb_sizeof_team", "gb_sizeof_args", "gb_sizeof_ctrl", "gb_sizeof_engine_config",
                 "gb_sizeof_launch", "gb_sizeof_switch"):
        getattr(L, name).restype = sz
        getattr(L, name).argtypes = []
    L.gb_payload_bytes.restype = sz
    L.gb_payload_bytes.argtypes = [i, i, sz]
    L.gb_symm_alloc.argtypes = [sz, ctypes.POINTER(vp)]
    L.gb_symm_free.argtypes = [vp]
    L.gb_symm_export.argtypes = [vp, ctypes.c_char_p]
    L.gb_symm_import.argtypes = [ctypes.c_char_p, ctypes.POINTER(vp)]
    L.gb_symm_unmap.argtypes = [vp]
    L.gb_can_access_peer.argtypes = [i, i, ctypes.POINTER(i)]
    L.gb_status_alloc.argtypes = [sz, ctypes.POINTER(vp)]
    L.gb_status_free.argtypes = [vp]
    L.gb_memset_async.argtypes = [vp, i, sz, vp]
    L.gb_launch_reduce.argtypes = [i, i, i, i, ctypes.POINTER(GbTeam), ctypes.POINTER(GbArgs),
                                   i, vp]
    L.gb_launch_copy.argtypes = [i, ctypes.POINTER(GbTeam), ctypes.POINTER(GbArgs), i, vp]
    L.gb_adamw_step.argtypes = [vp, vp, vp, vp, sz, vp] + [ctypes.c_float] * 6 + [i, vp]
    L.gb_adamw_span.argtypes = [vp, vp, vp, vp, sz, vp] + [ctypes.c_float] * 6 + [i, i, i, vp]
    L.gb_xent_fwd_bwd.argtypes = [vp, i, vp, sz, sz, sz, vp, vp, vp, vp]
    L.gb_allgather_gemm.argtypes = [ctypes.POINTER(GbTeam), vp, vp, vp, vp, vp, vp, ctypes.c_uint,
                                    i, i, i, sz, sz, i, i, vp]
    L.gb_allgather_gemm_pair.argtypes = L.gb_allgather_gemm.argtypes
    L.gb_gemm_reduce_scatter_bytes.restype = sz
    L.gb_gemm_reduce_scatter_bytes.argtypes = [i, i, i]
    L.gb_gemm_reduce_scatter.argtypes = [ctypes.POINTER(GbTeam), vp, vp, vp, vp, i, i, i, sz, sz,
                                         i, i, i, vp]
    L.gb_copy_to_host.argtypes = [vp, vp, sz, vp]
    L.gb_plan_hier.argtypes = [sz, i, i, i, i, sz, sz, sz, i, sz, i, i, i, ctypes.POINTER(GbHierPlanOut)]
    L.gb_engine_create.restype = vp
    L.gb_engine_create.argtypes = [ctypes.POINTER(GbTeam), ctypes.POINTER(GbEngineConfig)]
    L.gb_engine_destroy.restype = None
    L.gb_engine_destroy.argtypes = [vp]
    L.gb_engine_launches.restype = ctypes.c_ulonglong
    L.gb_engine_launches.argtypes = [vp]
    L.gb_engine_status.restype = ctypes.c_uint
    L.gb_engine_status.argtypes = [vp]
    launch = ctypes.POINTER(GbLaunch)
    L.gb_engine_prepare_all_reduce.argtypes = [vp, vp, vp, sz, i, i, i, i, launch]
    L.gb_engine_prepare_reduce_scatter.argtypes = [vp, vp, vp, sz, i, i, i, launch]
    L.gb_engine_prepare_all_gather.argtypes = [vp, vp, vp, sz, i, launch]
    L.gb_engine_prepare_broadcast.argtypes = [vp, vp, sz, i, i, launch]
    L.gb_engine_all_reduce.argtypes = [vp, vp, vp, sz, i, i, i, i, vp]
    L.gb_engine_reduce_scatter.argtypes = [vp, vp, vp, sz, i, i, i, vp]
    L.gb_engine_all_gather.argtypes = [vp, vp, vp, sz, i, vp]
    L.gb_engine_broadcast.argtypes = [vp, vp, sz, i, i, vp]
    L.gb_engine_barrier.argtypes = [vp, vp]
    ull = ctypes.c_ulonglong
    L.gb_device_synchronize.argtypes = []
    L.gb_mc_error_string.restype = ctypes.c_char_p
    L.gb_mc_error_string.argtypes = [i]
    L.gb_mc_supported.argtypes = [i, ctypes.POINTER(i)]
    L.gb_mc_granularity.argtypes = [i, i, sz, ctypes.POINTER(sz)]
    L.gb_mc_create.argtypes = [i, sz, ctypes.POINTER(ull)]
    L.gb_mc_add_device.argtypes = [ull, i]
    L.gb_mc_bind.argtypes = [ull, ull, sz]
    L.gb_mc_unbind.argtypes = [ull, i, sz]
    L.gb_vmm_create.argtypes = [i, sz, ctypes.POINTER(ull)]
    L.gb_vmm_release.argtypes = [ull]
    L.gb_vmm_export.argtypes = [ull, ctypes.POINTER(i)]
    L.gb_vmm_import.argtypes = [i, ctypes.POINTER(ull)]
    L.gb_vmm_map.argtypes = [ull, sz, sz, i, ctypes.POINTER(vp)]
    L.gb_vmm_unmap.argtypes = [vp, sz]
    L.gb_switch_plan.argtypes = [ctypes.POINTER(GbSwitch), i, sz, i, ctypes.POINTER(GbSwitchPlan)]
    L.gb_switch_all_reduce.argtypes = [ctypes.POINTER(GbTeam), ctypes.POINTER(GbSwitch), vp, vp, sz,
                                       i, i, i, vp]
    L.gb_switch_all_reduce_inplace.argtypes = [ctypes.POINTER(GbTeam), ctypes.POINTER(GbSwitch), sz, sz,
                                               i, i, i, vp]
    L.gb_engine_set_switch.argtypes = [vp, ctypes.POINTER(GbSwitch), ctypes.POINTER(GbSwitch), sz, i]
    L.gb_engine_set_switch_copy.argtypes = [vp, sz, sz]
    L.gb_engine_set_switch_oneshot.argtypes = [vp, sz]
    L.gb_engine_set_switch_oneshot.restype = None
    L.gb_switch_all_reduce_oneshot.argtypes = [ctypes.POINTER(GbTeam), ctypes.POINTER(GbSwitch), vp, vp, sz,
                                               i, i, i, vp]
    L.gb_engine_set_switch_copy.restype = None
    L.gb_switch_plan_copy.argtypes = [ctypes.POINTER(GbSwitch), i, sz, i, ctypes.POINTER(GbSwitchPlan)]
    L.gb_switch_reduce_scatter.argtypes = [ctypes.POINTER(GbTeam), ctypes.POINTER(GbSwitch), vp, vp, sz,
                                           i, i, i, vp]
    L.gb_switch_all_gather.argtypes = [ctypes.POINTER(GbTeam), ctypes.POINTER(GbSwitch), vp, vp, sz, i, vp]
    L.gb_switch_broadcast.argtypes = [ctypes.POINTER(GbTeam), ctypes.POINTER(GbSwitch), vp, sz, i, i, vp]
    L.gb_codec_quantize.argtypes = [i, i, i, vp, vp, vp, sz, vp]
    L.gb_codec_dequantize.argtypes = [i, i, i, vp, sz, i, vp, sz, vp]


def check(code: int, what: str) -> None:
    if code != 0:
        text = lib().gb_error_string(code).decode()
        raise RuntimeError(f"gpubridge native call {what} failed: {text} (CUDA error {code})")


def stream_ptr(device=None) -> int:
    return torch.cuda.current_stream(device).cuda_stream
