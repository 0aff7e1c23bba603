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


# ---- a pool of ranks that stays up for a whole test module ------------------------------------------
def _pool_entry(rank, world, vendors, path, env, mode, init, commands, results):
    """One pooled rank: join once, then run whatever the test process sends."""
    try:
        os.environ.update(env)
        if vendors[rank]:
            os.environ["GPUBRIDGE_VENDOR"] = vendors[rank]
            os.environ.setdefault("GPUBRIDGE_SIM_HOSTNAME", "simhost")
        else:
            os.environ["LOCAL_RANK"] = str(rank)
        torch.set_num_threads(1)
        import torch.distributed as dist

        import gpubridge_b200 as gb
        timeout = timedelta(seconds=40)
        warnings.simplefilter("ignore", gb.SplitTestWarning)
        if mode == "init":
            context = gb.init(f"file://{path}", rank=rank, world_size=world, timeout=timeout, **init)
        else:
            dist.init_process_group("gpubridge", init_method=f"file://{path}", rank=rank,
                                    world_size=world, timeout=timeout)
            context = world
        results.put((rank, "ready", None))
        while True:
            job = commands.get()
            if job is None:
                break
            fn, args = job
            try:
                results.put((rank, "ok", fn(rank, context, *args)))
            except BaseException as exc:  # noqa: BLE001
                results.put((rank, "error", f"{type(exc).__name__}: {exc}\n{traceback.format_exc()}"))
        if mode == "init":
            gb.destroy()
        else:
            dist.destroy_process_group()
    except BaseException as exc:  # noqa: BLE001
        results.put((rank, "error", f"{type(exc).__name__}: {exc}\n{traceback.format_exc()}"))


class RankPool:
    """Ranks that join once and then run many scenarios: ``pool.run(fn, *args)`` calls
    ``fn(rank, context, *args)`` on every rank (``context``: the topology in ``init`` mode, the
    world size in ``backend`` mode) and returns the results by rank.  Starting four processes
    and a process group costs seconds; a module of thirty scenarios pays it once.  After a
    failed scenario the group may be out of step, so the pool is rebuilt before the next one."""

    def __init__(self, vendors, directory, *, mode="backend", env=None, init=None):
        self.vendors, self.directory = list(vendors), str(directory)
        self.mode, self.env, self.init = mode, dict(env or {}), dict(init or {})
        self.procs, self.generation = [], 0
        self._start()

    def _start(self):
        global _counter
        _counter += 1
        self.generation += 1
        world = len(self.vendors)
        path = os.path.join(self.directory, f"pool-{os.getpid()}-{_counter}")
        ctx = mp.get_context("spawn")
        self.results = ctx.Queue()
        self.commands = [ctx.Queue() for _ in range(world)]
        self.procs = [ctx.Process(target=_pool_entry, args=(r, world, self.vendors, path, self.env,
                                                            self.mode, self.init, self.commands[r],
                                                            self.results))
                      for r in range(world)]
        for p in self.procs:
            p.start()
        self._collect(60, "ready")
        self.healthy = True

    def _collect(self, timeout, expect="ok"):
        world, got = len(self.vendors), {}
        try:
            for _ in range(world):
                rank, status, out = self.results.get(timeout=timeout)
                got[rank] = (status, out)
        except Exception:  # noqa: BLE001 - queue.Empty
            pass
        errors = [f"rank {r}: {out}" for r, (status, out) in sorted(got.items()) if status != expect]
        missing = [r for r in range(world) if r not in got]
        if missing:
            errors.append(f"ranks {missing} did not answer within {timeout} s")
        if errors:
            self.healthy = False
            raise AssertionError("\n".join(errors))
        return [got[r][1] for r in range(world)]

    def run(self, fn, *args, timeout=90):
        if not self.healthy:
            self.close(force=True)
            self._start()
        for queue in self.commands:
            queue.put((fn, args))
        return self._collect(timeout)

    def close(self, force=False):
        for queue in self.commands:
            try:
                queue.put(None)
            except Exception:  # noqa: BLE001
                pass
        for p in self.procs:
            p.join(1 if force else 15)
            if p.is_alive():
                p.kill()
        self.procs = []


def per_rank(rank, world, path, envs, init, fn=None, *args):
    """For ``run_ranks(..., mode="plain")``: set THIS rank's environment (``envs[rank]``), join
    with ``init`` and run ``fn(rank, topology, *args)`` - what a common ``env`` cannot express:
    ranks that were started with different settings."""
    import gpubridge_b200 as gb
    os.environ.update(envs.get(rank, {}))
    init = dict(init)
    seconds = init.pop("seconds", 40)
    with warnings.catch_warnings():
        warnings.simplefilter("ignore", gb.SplitTestWarning)
        topology = gb.init(f"file://{path}", rank=rank, world_size=world, timeout=timedelta(seconds=seconds), **init)
        try:
            return fn(rank, topology, *args) if fn is not None else "up"
        finally:
            gb.destroy()
