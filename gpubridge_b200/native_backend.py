"""``backend="gpubridge_native"``: the C++ front end of the ``torch.distributed`` backend.

    import gpubridge_b200.native_backend        # registers the name
    dist.init_process_group(backend="gpubridge_native")

or, for a program that already says ``backend="gpubridge"``: ``GPUBRIDGE_FRONT_END=native``.

torch wraps what :func:`create` returns - a ``c10d::Backend`` written in C++
(``csrc_torch/gb_c10d.cpp``) - in its own C++ ProcessGroup, so a collective on a CUDA tensor
goes dispatcher -> backend -> native engine -> kernel launch without running a line of Python:
the engine (``csrc/gb_engine.cu``) plans channels, chunking and grid and launches the fused
kernel on the team's communication stream, and the Work that comes back is an event behind
that launch.  ``all_reduce`` (SUM, AVG, MAX, MIN), ``broadcast``, ``all_gather_into_tensor``
and ``reduce_scatter_tensor`` take this path when the team has an NVLink fabric, the policy is
the default one and the bridge is not compressed.

Everything else is answered by the Python process group of ``backend="gpubridge"`` (one is
built per group and handed to the C++ object as its fallback), so the two names accept the
same programs: CPU tensors and CPU-only simulation, tensor lists, gather / scatter,
point-to-point, compressed or pipelined bridges, subgroups (HSDP), object collectives.
``GbBackend.native_calls`` / ``fallback_calls`` count which way calls went.

The Python-subclass backend of the reference (src/gpubridge/torch_backend.py) enters the
interpreter for every collective; here only the paths that are not latency-critical do.
"""
from __future__ import annotations

import threading

import torch.distributed as dist

from gpubridge_b200 import torch_backend as _python_backend

NAME = "gpubridge_native"

_lock = threading.Lock()
_made: dict[str, object] = {}        # group id -> backend: one object serves "cpu" and "cuda"
_python_groups: dict[str, object] = {}


def create(options, backend_options=None):
    """The creator torch calls once per device type of a new group."""
    from gpubridge_b200.ops import _build_c10d
    with _lock:
        backend = _made.get(options.group_id)
        if backend is None:
            fallback = _python_backend.create_python(options, backend_options)
            backend = _build_c10d.load().GbBackend(options.group_rank, options.group_size, fallback)
            _made[options.group_id] = backend
            _python_groups[options.group_id] = fallback
            fallback._on_shutdown = lambda key=options.group_id: forget(key)
        return backend


def backend_of(group=None):
    """The C++ backend object of ``group`` (default: the world), for its counters."""
    group = group or dist.distributed_c10d._get_default_group()
    with _lock:
        return _made.get(group.group_name)


def python_group_of(group=None):
    """The Python process group that answers what the C++ backend of ``group`` hands over."""
    group = group or dist.distributed_c10d._get_default_group()
    with _lock:
        return _python_groups.get(group.group_name)


def forget(group_id: str | None = None) -> None:
    """Drop the cache entry of a destroyed group (all of them by default)."""
    with _lock:
        for table in (_made, _python_groups):
            if group_id is None:
                table.clear()
            else:
                table.pop(group_id, None)


def register() -> None:
    """Make ``backend="gpubridge_native"`` known to ``torch.distributed`` (idempotent)."""
    if dist.is_available() and NAME not in dist.Backend.backend_list:
        dist.Backend.register_backend(NAME, create, extended_api=True, devices=["cpu", "cuda"])


register()
