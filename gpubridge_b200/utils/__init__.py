"""Small helpers shared by the benchmarks, the kit and user scripts.

    from gpubridge_b200.utils import ClockSampler, device_time, human_bytes, link_layout, parse_size
"""
from gpubridge_b200.config import parse_size
from gpubridge_b200.utils.clocks import ClockSampler
from gpubridge_b200.utils.links import link_layout
from gpubridge_b200.utils.timing import device_time, human_bytes, max_over_ranks

__all__ = ["ClockSampler", "device_time", "human_bytes", "link_layout", "max_over_ranks",
           "parse_size"]
