"""Which vendor a process belongs to, and a probe of what it can do that never raises
(reference: src/gpubridge/detect.py:18-108)."""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist

from gpubridge_b200.config import CPU_ONLY_ENV, VENDOR_ENV, VENDORS, _raw


def vendor_override() -> str | None:
    """``GPUBRIDGE_VENDOR`` if set (``nvidia``/``amd``), else None."""
    value = _raw(VENDOR_ENV).lower()
    if not value:
        return None
    if value not in VENDORS:
        raise ValueError(f"{VENDOR_ENV}={value!r} is not a known vendor; expected one of: "
                         f"{', '.join(VENDORS)}")
    return value


def detect_hardware_vendor() -> str:
    """The vendor of the installed torch build (a build is CUDA or ROCm, never both)."""
    if getattr(torch.version, "hip", None):
        return "amd"
    if getattr(torch.version, "cuda", None):
        return "nvidia"
    raise RuntimeError(
        "This PyTorch build has neither CUDA nor ROCm support, so the vendor cannot be detected "
        f"({CPU_ONLY_ENV} still needs a CUDA or ROCm build). To develop without GPUs, set "
        f"{VENDOR_ENV}=nvidia or {VENDOR_ENV}=amd to run in CPU simulation mode.")


def detect_vendor() -> str:
    return vendor_override() or detect_hardware_vendor()


@dataclass(frozen=True)
class Probe:
    """Build, GPUs and backends of one process.  A failed check leaves a safe default and a
    line in :attr:`errors`."""

    build_vendor: str | None
    torch_version: str
    cuda_version: str | None
    hip_version: str | None
    gpu_count: int
    nccl_available: bool
    gloo_available: bool
    errors: tuple[str, ...] = ()


def probe() -> Probe:
    errors: list[str] = []

    def attempt(label, fn, default):
        try:
            return fn()
        except Exception as exc:  # noqa: BLE001 - a probe must never take the process down
            errors.append(f"{label}: {type(exc).__name__}: {exc}")
            return default

    hip = attempt("torch.version.hip", lambda: getattr(torch.version, "hip", None), None)
    cuda = attempt("torch.version.cuda", lambda: getattr(torch.version, "cuda", None), None)
    fields = dict(
        build_vendor="amd" if hip else "nvidia" if cuda else None,
        torch_version=attempt("torch.__version__", lambda: str(torch.__version__), "unknown"),
        cuda_version=str(cuda) if cuda else None,
        hip_version=str(hip) if hip else None,
        gpu_count=attempt("torch.cuda.device_count", lambda: int(torch.cuda.device_count()), 0),
        nccl_available=attempt("dist.is_nccl_available", lambda: bool(dist.is_nccl_available()),
                               False),
        gloo_available=attempt("dist.is_gloo_available", lambda: bool(dist.is_gloo_available()),
                               False),
    )
    return Probe(errors=tuple(errors), **fields)
