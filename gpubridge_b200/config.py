"""Runtime settings: every environment variable the library reads, parsed in one place.

The variable names are the reference's (reference: src/gpubridge/config.py:16-49) so a
job script written for it keeps working.  Additions of this build are marked "B200".
Nothing here touches a device except :func:`resolve_config`, which only *queries*.
"""
from __future__ import annotations

import os
import socket
from dataclasses import dataclass

import torch

VENDORS = ("nvidia", "amd")

VENDOR_ENV = "GPUBRIDGE_VENDOR"                  # fake a vendor on CPU (simulation mode)
CPU_ONLY_ENV = "GPUBRIDGE_CPU_ONLY"              # CPU run, vendor from the torch build
SPLIT_TEST_ENV = "GPUBRIDGE_SPLIT_TEST"          # TEST ONLY: relabel part of a one-vendor job
SIM_HOSTNAME_ENV = "GPUBRIDGE_SIM_HOSTNAME"      # pretend host name (simulation only)
CHUNK_BYTES_ENV = "GPUBRIDGE_CHUNK_BYTES"        # pipelined policy chunk
THRESHOLDS_ENV = "GPUBRIDGE_THRESHOLDS"          # auto-tuned policy rules file
PINNED_STAGING_ENV = "GPUBRIDGE_PINNED_STAGING"  # host-staged bridge through pinned memory
BRIDGE_COMPRESSION_ENV = "GPUBRIDGE_BRIDGE_COMPRESSION"  # bf16 | fp8
POLICY_ENV = "GPUBRIDGE_POLICY"                  # torch backend: policy name
BRIDGE_ENV = "GPUBRIDGE_BRIDGE"                  # torch backend: bridge transport name
# ---- B200 additions -------------------------------------------------------------------
ISLANDS_ENV = "GPUBRIDGE_ISLANDS"                # "4,4" | "2,2,2,2" | "8": explicit island sizes
FABRIC_ENV = "GPUBRIDGE_FABRIC"                  # auto | off: NVLink symmetric-memory fast path
ALGO_ENV = "GPUBRIDGE_ALGO"                      # auto | one-shot | two-shot | nvls
CODEC_FORMAT_ENV = "GPUBRIDGE_CODEC_FORMAT"      # ref (256/pow2) | b200 (128/absmax)
WAIT_MS_ENV = "GPUBRIDGE_WAIT_TIMEOUT_MS"        # bound of every device-side wait
FABRIC_BYTES_ENV = "GPUBRIDGE_FABRIC_BYTES"      # symmetric workspace size per rank

SPLIT_TEST_MODES = ("half", "alternate", "node")
BRIDGE_COMPRESSION_MODES = ("bf16", "fp8")
CODEC_FORMATS = ("ref", "b200")
ALGOS = ("auto", "one-shot", "two-shot", "nvls")

CPU_BACKEND = "gloo"
GPU_BACKEND = "nccl"

_FALSE = ("", "0", "false", "no", "off")
_TRUE = ("1", "true", "yes", "on")
_UNITS = {"K": 1 << 10, "M": 1 << 20, "G": 1 << 30}


def _raw(name: str) -> str:
    return os.environ.get(name, "").strip()


def flag(name: str) -> bool:
    """A boolean variable; anything but a boolean word is a configuration error."""
    value = _raw(name).lower()
    if value in _FALSE:
        return False
    if value in _TRUE:
        return True
    raise ValueError(f"{name}={os.environ[name]!r} is not a boolean; use 1 or 0")


def choice(name: str, allowed: tuple[str, ...], default: str, *, off: bool = False) -> str:
    """One word out of ``allowed``.  With ``off`` the false words mean "not set" ("")."""
    value = _raw(name).lower()
    if off and value in (*_FALSE, "none"):
        return ""
    if not value:
        return default
    if value in allowed:
        return value
    raise ValueError(f"{name}={os.environ[name]!r} is not valid; use "
                     f"{' or '.join(allowed)}" + (", or leave it unset (off)" if off else ""))


def parse_size(text: str) -> int:
    """``"4M"``, ``"64K"``, ``"1G"``, ``"65536"`` (an optional trailing ``B``) to bytes."""
    value = text.strip().upper().removesuffix("B")
    try:
        if value and value[-1] in _UNITS:
            return int(float(value[:-1]) * _UNITS[value[-1]])
        return int(value)
    except ValueError:
        raise ValueError(f"{text!r} is not a size; use bytes or a K/M/G suffix, e.g. 4M") from None


def size_setting(name: str, default: int, *, multiple: int = 8) -> int:
    """A byte count that must be a positive multiple of ``multiple``."""
    raw = _raw(name)
    if not raw:
        return default
    try:
        value = parse_size(raw)
    except ValueError as exc:
        raise ValueError(f"{name}: {exc}") from None
    if value < multiple or value % multiple:
        raise ValueError(f"{name}={raw!r} must be a positive multiple of {multiple} bytes")
    return value


def is_cpu_only() -> bool:
    return flag(CPU_ONLY_ENV)


def pinned_staging_setting() -> bool:
    return flag(PINNED_STAGING_ENV)


def bridge_compression_setting() -> str:
    """``bf16``, ``fp8`` or ``""`` (off)."""
    return choice(BRIDGE_COMPRESSION_ENV, BRIDGE_COMPRESSION_MODES, "", off=True)


def codec_format_setting() -> str:
    """``ref``: 256 values per power-of-two scale (the reference's payload, bit for bit).
    ``b200``: 128 values per fp32 ``amax/448`` scale."""
    return choice(CODEC_FORMAT_ENV, CODEC_FORMATS, "ref")


def algo_setting() -> str:
    return choice(ALGO_ENV, ALGOS, "auto")


def fabric_setting() -> str:
    return choice(FABRIC_ENV, ("auto", "off"), "auto")


def wait_timeout_ms() -> int:
    raw = _raw(WAIT_MS_ENV)
    try:
        value = int(raw) if raw else 30_000
    except ValueError:
        raise ValueError(f"{WAIT_MS_ENV} must be a whole number of milliseconds") from None
    if value <= 0:
        raise ValueError(f"{WAIT_MS_ENV} must be positive")
    return value


def split_test_mode() -> str | None:
    value = _raw(SPLIT_TEST_ENV).lower()
    if value in _FALSE:
        return None
    if value in _TRUE:
        return "half"
    if value in SPLIT_TEST_MODES:
        return value
    raise ValueError(f"{SPLIT_TEST_ENV}={os.environ[SPLIT_TEST_ENV]!r} is not valid; use one of "
                     f"{', '.join(SPLIT_TEST_MODES)}, 1 (half) or 0 (off)")


def islands_setting() -> tuple[int, ...]:
    """Explicit island sizes, e.g. ``4,4``; empty when unset.  B200 addition: the
    reference's split modes only ever make two islands."""
    raw = _raw(ISLANDS_ENV)
    if not raw:
        return ()
    try:
        sizes = tuple(int(part) for part in raw.replace("+", ",").split(","))
    except ValueError:
        raise ValueError(f"{ISLANDS_ENV}={raw!r} must be island sizes such as 4,4") from None
    if not sizes or min(sizes) <= 0:
        raise ValueError(f"{ISLANDS_ENV}={raw!r} must be positive island sizes such as 4,4")
    return sizes


def chunk_bytes_setting(default: int) -> int:
    return size_setting(CHUNK_BYTES_ENV, default)


def is_simulated() -> bool:
    """CPU run with Gloo islands: a faked vendor or CPU-only mode."""
    return bool(_raw(VENDOR_ENV)) or is_cpu_only()


def hostname(simulated: bool) -> str:
    if simulated and _raw(SIM_HOSTNAME_ENV):
        return _raw(SIM_HOSTNAME_ENV)
    return socket.gethostname()


@dataclass(frozen=True)
class Config:
    """Where and how this process communicates."""

    simulated: bool
    island_backend: str
    device: torch.device


def resolve_config() -> Config:
    """Island backend and device of this rank (reference: config.py:193-236).

    GPU ranks use ``cuda:$LOCAL_RANK`` (the current device without it).  Only in a split
    test may the index wrap around the visible GPUs.  A bad index is an error *here*, so
    discovery can report it from every rank instead of one rank dying in ``set_device``.
    """
    if is_simulated():
        return Config(True, CPU_BACKEND, torch.device("cpu"))
    if not torch.cuda.is_available():
        raise RuntimeError(
            "No GPU is visible to this process. To develop without GPUs, set "
            f"{VENDOR_ENV}=nvidia or {VENDOR_ENV}=amd (CPU simulation), or {CPU_ONLY_ENV}=1.")
    local_rank = os.environ.get("LOCAL_RANK")
    if local_rank is None:
        index = torch.cuda.current_device()
    else:
        try:
            index = int(local_rank)
        except ValueError:
            raise RuntimeError(f"LOCAL_RANK={local_rank!r} is not an integer; the launcher "
                               "(torchrun, srun) sets it") from None
    count = torch.cuda.device_count()
    if count and index >= count and (split_test_mode() is not None or islands_setting()):
        index %= count
    if not 0 <= index < count:
        asked = f"LOCAL_RANK={local_rank}" if local_rank is not None else "The current device"
        raise RuntimeError(
            f"{asked} asks for GPU {index}, but this process sees only {count} GPU(s). Start "
            "no more processes per node than it has GPUs (torchrun --nproc-per-node) and check "
            "CUDA_VISIBLE_DEVICES.")
    return Config(False, GPU_BACKEND, torch.device("cuda", index))


def gpu_identity(device: torch.device) -> str | None:
    """UUID and PCI address of the GPU behind ``device``: equal in every process that drives
    it, unlike the index.  None on CPU, ``""`` when the GPU reports neither."""
    if device.type != "cuda":
        return None
    try:
        props = torch.cuda.get_device_properties(device)
    except Exception:  # noqa: BLE001 - informational only
        return ""
    parts = []
    uuid = str(getattr(props, "uuid", "") or "")
    if uuid.strip("0-"):
        parts.append(f"uuid {uuid}")
    pci = [getattr(props, f"pci_{n}_id", None) for n in ("domain", "bus", "device")]
    if None not in pci and any(pci):
        parts.append("pci {:04x}:{:02x}:{:02x}".format(*pci))
    return ", ".join(parts)
