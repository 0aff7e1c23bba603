"""What NVML says about the NVLink side of this machine - read-only.

    layout = link_layout()        # None when NVML or the GPUs are not there
    layout["gpus"][0] == {"index": 0, "links_active": 18, "link_version": 5, "to_switch": 18, "to_gpu": 0, ...}
    layout["fabric"] == "nvswitch"   # every active link of every GPU ends at a switch

Only getters are called (link state, link version, remote device type, names): nothing here
changes a setting of a GPU.  The fused kernels do not need this to run - peer access between
every pair is what they need, and the fabric checks that itself - but a box whose GPUs are
joined pairwise by direct links, or that lost links, behaves differently from an NVSwitch box
(every peer at full rate, in-switch reduction), and the probe and the records say which one
a number was measured on.  The reference has no link discovery (its islands are vendor
labels); this is the "discovers the GPU / NVLink / NVSwitch layout" part of detection.
"""
from __future__ import annotations

from typing import Any

MAX_LINKS = 18
REMOTE_GPU, REMOTE_IBMNPU, REMOTE_SWITCH = 0, 1, 2


def link_layout(nvml: Any = None) -> dict | None:
    """Per GPU: active links, their version, how many end at a switch and how many at a GPU;
    and the machine's kind: ``nvswitch``, ``direct`` (GPU-to-GPU links), ``mixed`` or ``none``.
    ``nvml``: a module with pynvml's functions (tests pass a fake); default: pynvml."""
    try:
        if nvml is None:
            import pynvml as nvml
        nvml.nvmlInit()
    except Exception:  # noqa: BLE001 - no NVML: nothing to say
        return None
    try:
        gpus = []
        for index in range(nvml.nvmlDeviceGetCount()):
            handle = nvml.nvmlDeviceGetHandleByIndex(index)
            name = nvml.nvmlDeviceGetName(handle)
            entry = {"index": index, "name": name.decode() if isinstance(name, bytes) else str(name),
                     "links_active": 0, "link_version": None, "to_switch": 0, "to_gpu": 0, "to_other": 0}
            for link in range(getattr(nvml, "NVML_NVLINK_MAX_LINKS", MAX_LINKS)):
                try:
                    if not nvml.nvmlDeviceGetNvLinkState(handle, link):
                        continue
                except Exception:  # noqa: BLE001 - a link this GPU does not have
                    continue
                entry["links_active"] += 1
                try:
                    entry["link_version"] = int(nvml.nvmlDeviceGetNvLinkVersion(handle, link))
                except Exception:  # noqa: BLE001
                    pass
                try:
                    remote = int(nvml.nvmlDeviceGetNvLinkRemoteDeviceType(handle, link))
                except Exception:  # noqa: BLE001
                    remote = -1
                key = "to_switch" if remote == REMOTE_SWITCH else "to_gpu" if remote == REMOTE_GPU else "to_other"
                entry[key] += 1
            gpus.append(entry)
        active = sum(g["links_active"] for g in gpus)
        to_switch, to_gpu = sum(g["to_switch"] for g in gpus), sum(g["to_gpu"] for g in gpus)
        fabric = ("none" if active == 0 else "nvswitch" if to_switch == active
                  else "direct" if to_gpu == active else "mixed")
        uneven = len({g["links_active"] for g in gpus}) > 1
        return {"gpus": gpus, "fabric": fabric, "links_uneven": uneven}
    finally:
        try:
            nvml.nvmlShutdown()
        except Exception:  # noqa: BLE001
            pass
