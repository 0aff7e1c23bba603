"""Run one function on several CPU ranks (simulation mode: Gloo islands, faked vendors).

Every rank is a spawned process that sets ``GPUBRIDGE_VENDOR`` to its entry of ``vendors``,
joins through a ``file://`` rendezvous and calls ``fn``.  Failures come back as text and
fail the test; a rank that hangs is killed after ``timeout`` seconds.  Exactness trick used
throughout (the reference's: tests/_harness.py:92-105): integer-valued data, so a sum is
exact in any order and any dtype.

``mode="init"``   ``gpubridge_b200.init(**init)`` then ``fn(rank, topology, *args)``
``mode="backend"`` ``dist.init_process_group("gpubridge")`` then ``fn(rank, world, *args)``
``mode="raw"``    nothing: ``fn(rank, world, path, *args)`` joins by itself
"""
from __future__ import annotations

import os
import traceback
import warnings
from datetime import timedelta

import torch
import torch.multiprocessing as mp


def rank_tensor(rank: int, numel: int, dtype=torch.float32) -> torch.Tensor:
    """Integer-valued, different on every rank, small enough to stay exact in bf16 sums."""
    return ((torch.arange(numel) % 7) + rank - 3).to(dtype)


def expected_sum(world: int, numel: int, dtype=torch.float32) -> torch.Tensor:
    return sum(rank_tensor(r, numel, torch.float64) for r in range(world)).to(dtype)


def _entry(rank, world, vendors, fn, path, env, args, mode, init, results):
    try:
        os.environ.update(env)
        if vendors[rank]:
            os.environ["GPUBRIDGE_VENDOR"] = vendors[rank]
            os.environ.setdefault("GPUBRIDGE_SIM_HOSTNAME", "simhost")
        else:                       # a real GPU rank: one process per GPU
            os.environ["LOCAL_RANK"] = str(rank)
        torch.set_num_threads(1)
        import torch.distributed as dist

        import gpubridge_b200 as gb
        timeout = timedelta(seconds=40)
        with warnings.catch_warnings():
            warnings.simplefilter("ignore", gb.SplitTestWarning)
            if mode == "init":
                topology = gb.init(f"file://{path}", rank=rank, world_size=world,
                                   timeout=timeout, **init)
                try:
                    out = fn(rank, topology, *args)
                finally:
                    gb.destroy()
            elif mode in ("backend", "native-backend"):
                if mode == "native-backend":
                    import gpubridge_b200.native_backend  # noqa: F401 - registers the name
                dist.init_process_group("gpubridge" if mode == "backend" else "gpubridge_native",
                                        init_method=f"file://{path}", rank=rank,
                                        world_size=world, timeout=timeout)
                try:
                    out = fn(rank, world, *args)
                finally:
                    dist.destroy_process_group()
            else:
                out = fn(rank, world, path, *args)
        results.put((rank, "ok", out))
    except BaseException as exc:  # noqa: BLE001
        results.put((rank, "error", f"{type(exc).__name__}: {exc}\n{traceback.format_exc()}"))


_counter = 0


def run_ranks(vendors, fn, tmp_path, *args, env=None, mode="init", init=None, timeout=90,
              expect_error=None):
    """Run ``fn`` on ``len(vendors)`` ranks and return each rank's result, by rank.  With
    ``expect_error`` (a regex) every rank must fail with a matching message instead."""
    global _counter
    _counter += 1
    world = len(vendors)
    path = os.path.join(str(tmp_path), f"rdzv-{os.getpid()}-{_counter}")
    ctx = mp.get_context("spawn")
    results = ctx.Queue()
    procs = [ctx.Process(target=_entry, args=(r, world, list(vendors), fn, path, dict(env or {}),
                                              args, mode, dict(init or {}), results))
             for r in range(world)]
    for p in procs:
        p.start()
    got = {}
    try:
        for _ in range(world):
            rank, status, out = results.get(timeout=timeout)
            got[rank] = (status, out)
    except Exception:  # noqa: BLE001 - queue.Empty: a rank hung
        pass
    for p in procs:
        p.join(5)
        if p.is_alive():
            p.kill()
    missing = [r for r in range(world) if r not in got]
    if expect_error is not None:
        import re
        assert not missing, f"ranks {missing} did not finish within {timeout} s"
        for r, (status, out) in sorted(got.items()):
            assert status == "error", f"rank {r} was expected to fail but returned {out!r}"
            assert re.search(expect_error, out), f"rank {r} failed differently:\n{out}"
        return [got[r][1] for r in range(world)]
    errors = [f"rank {r}: {out}" for r, (status, out) in sorted(got.items()) if status != "ok"]
    if missing:
        errors.append(f"ranks {missing} did not finish within {timeout} s")
    if errors:
        raise AssertionError("\n".join(errors))
    return [got[r][1] for r in range(world)]


TWO_BY_TWO = ("nvidia", "nvidia", "amd", "amd")
def gpu_ranks(world: int):
    """``vendors`` for ``world`` real GPU ranks (the vendor comes from the torch build)."""
    return ("",) * world


LAYOUTS = {
    "2+2": TWO_BY_TWO,
    "interleaved": ("nvidia", "amd", "nvidia", "amd"),
    "3+1": ("nvidia", "nvidia", "nvidia", "amd"),
    "1+3": ("nvidia", "amd", "amd", "amd"),
    "single-vendor": ("nvidia", "nvidia", "nvidia"),
    "single-rank": ("amd",),
}
