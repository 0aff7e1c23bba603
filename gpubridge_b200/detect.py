"""Vendor of this process and a survey of what it can do.

Two questions are answered here.  *Which island label does this rank carry?*  An explicit
``GPUBRIDGE_VENDOR`` wins (that is how CPU simulation and the split tests relabel ranks);
otherwise the label follows the torch build, which is compiled for exactly one GPU runtime.
*What is installed?*  :func:`probe` collects versions, the GPU count, the collective backends
and - on a CUDA build - the first GPU's compute capability, and turns every failure into a
line of text instead of an exception, because it runs inside bug reports and preflight checks
where a crash would hide the very thing being looked for.  Public names and the fields of
:class:`Probe` match the reference (src/gpubridge/detect.py) so reports stay comparable.
"""
from __future__ import annotations

import dataclasses

import torch
import torch.distributed as dist

from gpubridge_b200 import config as _config

# torch.version attribute that is non-empty on a build for that vendor, in lookup order
_BUILD_MARKERS = (("amd", "hip"), ("nvidia", "cuda"))


def _build_vendor() -> str | None:
    for vendor, marker in _BUILD_MARKERS:
        if getattr(torch.version, marker, None):
            return vendor
    return None


def vendor_override() -> str | None:
    """The label forced by ``GPUBRIDGE_VENDOR``, or None when the variable is empty.  An
    unknown label is an error rather than a silent third island."""
    forced = _config._raw(_config.VENDOR_ENV).lower()
    if forced and forced not in _config.VENDORS:
        known = ", ".join(_config.VENDORS)
        raise ValueError(f"{_config.VENDOR_ENV}={forced!r} is not a known vendor; expected one of: {known}")
    return forced or None


def detect_hardware_vendor() -> str:
    """The vendor the installed torch was built for."""
    vendor = _build_vendor()
    if vendor is not None:
        return vendor
    raise RuntimeError(
        "This PyTorch build has neither CUDA nor ROCm support, so there is no vendor to detect "
        f"(and {_config.CPU_ONLY_ENV} does not change that: it still wants a GPU build). "
        f"For development without GPUs set {_config.VENDOR_ENV}=nvidia or "
        f"{_config.VENDOR_ENV}=amd, which selects CPU simulation mode.")


def detect_vendor() -> str:
    return vendor_override() or detect_hardware_vendor()


@dataclasses.dataclass(frozen=True)
class Probe:
    """What :func:`probe` found.  A check that failed keeps its neutral default and leaves a
    line in ``errors``."""

    build_vendor: str | None
    torch_version: str
    cuda_version: str | None
    hip_version: str | None
    gpu_count: int
    nccl_available: bool
    gloo_available: bool
    errors: tuple[str, ...] = ()
    compute_capability: str | None = None        # of GPU 0, e.g. "10.0" on a B200


def _capability() -> str | None:
    if not torch.cuda.is_available():
        return None
    major, minor = torch.cuda.get_device_capability(0)
    return f"{major}.{minor}"


# field -> (what to evaluate, what to report when that raises)
_CHECKS = {
    "torch_version": (lambda: str(torch.__version__), "unknown"),
    "cuda_version": (lambda: (str(torch.version.cuda) if getattr(torch.version, "cuda", None) else None), None),
    "hip_version": (lambda: (str(torch.version.hip) if getattr(torch.version, "hip", None) else None), None),
    "build_vendor": (_build_vendor, None),
    "gpu_count": (lambda: int(torch.cuda.device_count()), 0),
    "nccl_available": (lambda: bool(dist.is_nccl_available()), False),
    "gloo_available": (lambda: bool(dist.is_gloo_available()), False),
    "compute_capability": (_capability, None),
}


def probe() -> Probe:
    """Survey this process.  Never raises."""
    found: dict[str, object] = {}
    problems: list[str] = []
    for field, (evaluate, neutral) in _CHECKS.items():
        try:
            found[field] = evaluate()
        except Exception as failure:  # noqa: BLE001 - the whole point: report, do not crash
            found[field] = neutral
            problems.append(f"{field}: {type(failure).__name__}: {failure}")
    return Probe(errors=tuple(problems), **found)
