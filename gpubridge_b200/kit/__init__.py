"""Validation kit: what the per-rank check, gate and benchmark programs share.

Covers the ground of the reference's ``scripts/gpu/gpukit.py`` (Record :366-418, redaction
:76-102, environment :289-321, run_info :324-355, queue_gpu_delay :521-541): a journal that
is rewritten after every stage so that a crash or hang shows where a rank stopped; strings
scrubbed of home directories, user names and URL credentials before they reach disk; a
description of the machine and of how the run formed its islands; and a way to queue a known
amount of GPU work without BLAS.

    journal = Journal(out / f"rank{rank}.json", "check")
    with journal.stage("init") as entry:
        ...
        entry["ok"] = False          # a failed check; exceptions mark the stage failed too
    sys.exit(journal.close())
"""
from __future__ import annotations

import contextlib
import faulthandler
import getpass
import json
import os
import platform
import re
import socket
import sys
import time
import traceback
from dataclasses import asdict
from pathlib import Path
from typing import Any, Iterator

import torch

KIT_VERSION = 1

#: Variables worth recording, by exact name or prefix; anything that smells like a secret is
#: left out even if it matches.
_ENV_NAMES = ("RANK", "LOCAL_RANK", "WORLD_SIZE", "MASTER_ADDR", "MASTER_PORT",
              "CUDA_VISIBLE_DEVICES", "OMP_NUM_THREADS")
_ENV_PREFIXES = ("GPUBRIDGE_", "NCCL_", "GLOO_", "TORCH_NCCL_", "KIT_")
_SECRET = ("TOKEN", "SECRET", "PASSWORD", "PASSWD", "KEY", "CREDENTIAL")


def redact(text: str) -> str:
    """``text`` with URL credentials, the home directory and the user name (as a path
    component) replaced by placeholders."""
    stop = r"(?=/|$|\s|['\":,])"
    text = re.sub(r"(\w+://)[^/@\s]+@", r"\1***@", text)
    home = os.path.expanduser("~").rstrip("/")
    if len(home) > 1:
        text = re.sub(re.escape(home) + stop, "~", text)
    try:
        user = getpass.getuser()
    except Exception:               # uid without a name, in some containers
        user = ""
    if user and user != "root":
        text = re.sub(f"/{re.escape(user)}{stop}", "/$USER", text)
    return text


def scrub(data: Any) -> Any:
    if isinstance(data, str):
        return redact(data)
    if isinstance(data, dict):
        return {str(k): scrub(v) for k, v in data.items()}
    if isinstance(data, (list, tuple)):
        return [scrub(v) for v in data]
    return data


def recorded_env(environ: dict[str, str] | None = None) -> dict[str, str]:
    environ = dict(os.environ) if environ is None else environ
    return {k: redact(v) for k, v in sorted(environ.items())
            if (k in _ENV_NAMES or k.startswith(_ENV_PREFIXES))
            and not any(word in k.upper() for word in _SECRET)}


def _try(fn, default=None):
    try:
        return fn()
    except Exception:
        return default


def device_info(index: int) -> dict[str, Any]:
    props = torch.cuda.get_device_properties(index)
    return {"index": index, "name": props.name,
            "capability": f"{props.major}.{props.minor}",
            "memory_bytes": props.total_memory, "sms": props.multi_processor_count,
            "pci_bus_id": _try(lambda: f"{props.pci_bus_id:02x}:{props.pci_device_id:02x}")}


def environment() -> dict[str, Any]:
    """The machine and software of this process."""
    import gpubridge_b200 as gb
    has_gpu = torch.cuda.is_available()
    count = torch.cuda.device_count() if has_gpu else 0
    return scrub({
        "hostname": socket.gethostname(), "platform": platform.platform(),
        "python": platform.python_version(), "pid": os.getpid(),
        "gpubridge_b200": gb.__version__, "torch": torch.__version__,
        "torch_cuda": torch.version.cuda,
        "nccl": _try(lambda: ".".join(map(str, torch.cuda.nccl.version()))),
        "cuda_available": has_gpu, "device_count": count,
        "devices": [_try(lambda i=i: device_info(i)) for i in range(count)],
        "nvlink_fabric": _try(_nvlink_fabric) if has_gpu else None,
        "probe": _try(lambda: asdict(gb.probe())),
        "native_library": _try(_native_library),
        "env": recorded_env(),
    })


def _nvlink_fabric() -> str | None:
    """``nvswitch`` / ``direct`` / ``mixed`` / ``none`` as NVML reports it (read-only)."""
    from gpubridge_b200.utils.links import link_layout
    layout = link_layout()
    return None if layout is None else layout["fabric"]


def _native_library() -> dict[str, Any]:
    from gpubridge_b200.ops import _build
    return {"path": os.path.basename(_build.LIB), "built": os.path.exists(_build.LIB)}


def run_info(topology) -> dict[str, Any]:
    """How the run was set up; a relabelled single-vendor run is never mistaken for a
    mixed-vendor one."""
    fabric = topology.fabric
    info = {
        "kind": topology.run_kind, "split_test": topology.split_test,
        "real_mixed_vendor": topology.run_kind == "gpu-mixed",
        "world_size": topology.world_size, "rank": topology.rank,
        "vendor_label": topology.vendor, "detected_vendor": topology.detected_vendor,
        "device": str(topology.device),
        "islands": [{"vendor": i.vendor, "ranks": list(i.ranks), "leader": i.leader}
                    for i in topology.layout.islands],
        "bridge": topology.peers[topology.rank].bridge, "policy": topology.policy_name,
        "pinned_staging": topology.pinned_staging,
        "fused": fabric is not None,
        "fabric_bytes": getattr(fabric, "nbytes", None),
    }
    if topology.split_test:
        info["warning"] = ("SPLIT TEST: the islands are relabelled ranks of one vendor; "
                           "this is not a mixed-vendor result.")
    return info


def write_json(path: Path, data: dict[str, Any]) -> None:
    """Atomic (write beside, then rename), every string scrubbed."""
    path.parent.mkdir(parents=True, exist_ok=True)
    tmp = path.with_suffix(path.suffix + ".tmp")
    tmp.write_text(json.dumps(scrub(json.loads(json.dumps(data, default=str))), indent=2))
    tmp.replace(path)


class Journal:
    """A rank's record of a kit program, rewritten after every stage.

    A stage whose ``ok`` is still ``None`` on disk is the one the rank was in when it died or
    hung; after ``hang_dump_seconds`` inside one stage every thread's stack goes to
    ``<name>.stacks.txt`` beside the record."""

    def __init__(self, path: Path, program: str, *, hang_dump_seconds: float = 600.0) -> None:
        self.path = Path(path)
        self.path.parent.mkdir(parents=True, exist_ok=True)
        self._stacks = open(self.path.with_suffix(".stacks.txt"), "w")  # noqa: SIM115
        self._hang = hang_dump_seconds
        self.failed = False
        self.data: dict[str, Any] = {
            "kit_version": KIT_VERSION, "program": program, "argv": list(sys.argv),
            "started": time.strftime("%Y-%m-%dT%H:%M:%S%z"), "environment": environment(),
            "run": None, "stages": [], "ok": None,
        }
        self.flush()

    def flush(self) -> None:
        write_json(self.path, self.data)

    @contextlib.contextmanager
    def stage(self, name: str) -> Iterator[dict[str, Any]]:
        entry: dict[str, Any] = {"name": name, "ok": None}
        self.data["stages"].append(entry)
        self.flush()
        if self._hang > 0:
            faulthandler.dump_traceback_later(self._hang, file=self._stacks)
        t0 = time.monotonic()
        try:
            yield entry
        except BaseException:
            entry["ok"] = False
            entry["error"] = traceback.format_exc()
            raise
        else:
            if entry["ok"] is None:
                entry["ok"] = True
        finally:
            if self._hang > 0:
                faulthandler.cancel_dump_traceback_later()
            entry["seconds"] = round(time.monotonic() - t0, 4)
            self.failed = self.failed or not entry["ok"]
            self.flush()

    def close(self) -> int:
        """Record the overall result; returns the process exit code."""
        self.data["ok"] = not self.failed
        self.data["finished"] = time.strftime("%Y-%m-%dT%H:%M:%S%z")
        self.flush()
        self._stacks.close()
        return 0 if self.data["ok"] else 1


def rank_from_env() -> int:
    return int(os.environ.get("RANK", "0"))


def default_timeout(fallback: float) -> float:
    try:
        return float(os.environ.get("KIT_TIMEOUT", "")) or fallback
    except ValueError:
        return fallback


def sync(device: torch.device) -> None:
    if device.type == "cuda":
        torch.cuda.synchronize(device)


_CYCLES_PER_SECOND: dict[int, float] = {}


def queue_gpu_delay(device: torch.device, seconds: float) -> None:
    """Queue roughly ``seconds`` of work on the current stream without waiting for it:
    torch's spin kernel, calibrated once per device against CUDA events.  What is queued
    behind it on the stream starts only when it ends.  Nothing happens on CPU."""
    if device.type != "cuda" or seconds <= 0:
        return
    index = device.index if device.index is not None else torch.cuda.current_device()
    with torch.cuda.device(index):
        if index not in _CYCLES_PER_SECOND:
            probe = 20_000_000
            torch.cuda._sleep(1000)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            torch.cuda._sleep(probe)
            b.record()
            b.synchronize()
            _CYCLES_PER_SECOND[index] = probe / max(a.elapsed_time(b) * 1e-3, 1e-6)
        torch.cuda._sleep(max(1, int(_CYCLES_PER_SECOND[index] * seconds)))


__all__ = ["Journal", "KIT_VERSION", "default_timeout", "device_info", "environment",
           "queue_gpu_delay", "rank_from_env", "recorded_env", "redact", "run_info", "scrub",
           "sync", "write_json"]
