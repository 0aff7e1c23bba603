"""SM clocks and throttle reasons while a timed region runs.

A measurement is only as good as the clocks it ran at: a region that saw a hardware or thermal
slowdown, or clocks stuck far below the maximum with no reason given (a leftover clock lock),
should be taken again.  ``ClockSampler`` polls ``nvidia-smi`` in the background (it only
reads; it never changes a GPU setting) and summarises what it saw.

    sampler = ClockSampler(device_index); sampler.start()
    ... timed region ...
    clocks = sampler.stop()      # {"sm_mhz": median, "sm_max_mhz": ..., "samples": n, "reasons": [...]}
"""
from __future__ import annotations

import statistics
import subprocess
import threading

QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
REASONS = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
#: reasons that invalidate a measurement (a power cap during dense GEMMs is normal)
REJECT = frozenset(REASONS[:3])


def summarise(lines: list[str]) -> dict:
    """The summary of ``nvidia-smi --format=csv,noheader,nounits`` lines of :data:`QUERY`."""
    clocks, top, reasons = [], None, set()
    for line in lines:
        parts = [p.strip() for p in line.split(",")]
        if len(parts) < 9:
            continue
        try:
            clocks.append(float(parts[1]))
            top = float(parts[2])
        except ValueError:
            continue
        for name, value in zip(REASONS, parts[5:9]):
            if value.lower().startswith("active"):
                reasons.add(name)
    return {"sm_mhz": statistics.median(clocks) if clocks else None, "sm_max_mhz": top,
            "samples": len(clocks), "reasons": sorted(reasons)}


def acceptable(summary: dict, floor: float = 0.5) -> bool:
    """False when the region saw a slowdown, or clocks below ``floor`` of the maximum with no
    reason at all."""
    if REJECT & set(summary.get("reasons", ())):
        return False
    sm, top = summary.get("sm_mhz"), summary.get("sm_max_mhz")
    if sm and top and sm < floor * top and not summary.get("reasons"):
        return False
    return True


class ClockSampler:
    def __init__(self, index: int, period_ms: int = 100) -> None:
        self.index, self.period_ms, self.lines, self.proc = index, period_ms, [], None

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={QUERY}", "--format=csv,noheader,nounits",
                 "-lms", str(self.period_ms), "-i", str(self.index)], stdout=subprocess.PIPE,
                stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self) -> None:
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "samples": 0,
                    "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        return summarise(self.lines)
