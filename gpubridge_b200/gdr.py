"""Making data a network adapter wrote into GPU memory visible to kernels.

When an adapter writes straight into device memory (GPUDirect RDMA), a kernel launched after
the receive completed may still not see the bytes unless the writes are flushed - or the
device promises an ordering that makes the flush unnecessary.  This module decides which, once
per device, and carries out the flush when one is needed (the reference does the same for its
UCX and verbs bridges: ucx/gdr.py:78-109).

    plan = gdr.plan(device_index)        # cached per device
    ... receive completed ...
    plan.after_receive()                 # a driver call, or nothing

The decision reads three driver attributes of the device:

* GPUDirect RDMA supported at all - if not, nothing is ever written directly, no flush;
* the write ordering the device guarantees: ``owner`` or wider means a kernel of the owning
  context sees completed writes without help - no flush;
* otherwise the flush options must include "host" (the flush is a host-side driver call), else
  direct receives are refused on this device and callers must stage through host memory.

The driver is reached through ``cuda-python`` when present; tests hand in a fake with the same
three calls.  Nothing here touches a device setting.
"""
from __future__ import annotations

import dataclasses
import threading
from typing import Any, Callable

ORDER_NONE, ORDER_OWNER, ORDER_ALL = 0, 100, 200
FLUSH_VIA_HOST = 1


@dataclasses.dataclass(frozen=True)
class FlushPlan:
    device: int
    direct_ok: bool
    """Whether receiving straight into this device's memory is allowed at all."""
    flush_needed: bool
    reason: str
    _flush: Callable[[], None] | None = None

    def after_receive(self) -> None:
        """Call after a direct receive completed and before a kernel reads the data."""
        if self.flush_needed and self._flush is not None:
            self._flush()

    def describe(self) -> dict:
        return {"device": self.device, "direct_ok": self.direct_ok,
                "flush_needed": self.flush_needed, "reason": self.reason}


class CudaDriver:
    """The three driver calls the decision needs, through ``cuda-python``."""

    def __init__(self) -> None:
        try:
            from cuda.bindings import driver          # cuda-python >= 12.6 layout
        except ImportError:                           # pragma: no cover - older layout
            from cuda import cuda as driver
        self.api = driver
        self._check(driver.cuInit(0))

    @staticmethod
    def _check(result) -> Any:
        code, *rest = result if isinstance(result, tuple) else (result,)
        if int(code) != 0:
            raise RuntimeError(f"CUDA driver call failed with code {int(code)}")
        return rest[0] if rest else None

    def attribute(self, device: int, name: str) -> int:
        handle = self._check(self.api.cuDeviceGet(device))
        which = getattr(self.api.CUdevice_attribute, f"CU_DEVICE_ATTRIBUTE_{name}")
        return int(self._check(self.api.cuDeviceGetAttribute(which, handle)))

    def flush_owner(self) -> None:
        target = self.api.CUflushGPUDirectRDMAWritesTarget.CU_FLUSH_GPU_DIRECT_RDMA_WRITES_TARGET_CURRENT_CTX
        scope = self.api.CUflushGPUDirectRDMAWritesScope.CU_FLUSH_GPU_DIRECT_RDMA_WRITES_TO_OWNER
        self._check(self.api.cuFlushGPUDirectRDMAWrites(target, scope))


def decide(device: int, driver) -> FlushPlan:
    """The plan for one device from a driver object (``attribute(device, name)``,
    ``flush_owner()``).  Pure apart from the attribute reads."""
    try:
        supported = driver.attribute(device, "GPU_DIRECT_RDMA_SUPPORTED")
    except Exception as failure:  # noqa: BLE001 - an old driver: treat as unsupported
        return FlushPlan(device, False, False, f"the driver cannot say ({failure}); receive through host memory")
    if not supported:
        return FlushPlan(device, False, False, "GPUDirect RDMA is not supported on this device")
    ordering = driver.attribute(device, "GPU_DIRECT_RDMA_WRITES_ORDERING")
    if ordering >= ORDER_OWNER:
        scope = "every device" if ordering >= ORDER_ALL else "the owning context"
        return FlushPlan(device, True, False, f"completed writes are ordered for {scope}: no flush")
    options = driver.attribute(device, "GPU_DIRECT_RDMA_FLUSH_WRITES_OPTIONS")
    if options & FLUSH_VIA_HOST:
        return FlushPlan(device, True, True, "writes are unordered: flushed by a driver call after each receive",
                         driver.flush_owner)
    return FlushPlan(device, False, False,
                     "writes are unordered and this device offers no host-side flush: receive through host memory")


_plans: dict[int, FlushPlan] = {}
_lock = threading.Lock()


def plan(device: int, driver=None) -> FlushPlan:
    """The cached plan of ``device``; ``driver`` overrides the real one (tests)."""
    if driver is not None:
        return decide(device, driver)
    with _lock:
        if device not in _plans:
            try:
                _plans[device] = decide(device, CudaDriver())
            except Exception as failure:  # noqa: BLE001 - no driver here (CPU box)
                _plans[device] = FlushPlan(device, False, False, f"no CUDA driver: {failure}")
        return _plans[device]
