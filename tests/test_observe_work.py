"""Observers, in_flight, the async queue and failure poisoning in CPU simulation (reference:
tests/test_observe.py, test_work_queue.py, test_hot_path.py)."""
import pytest
import torch

from _harness import TWO_BY_TWO, expected_sum, rank_tensor, run_ranks


def _observe(rank, topology):
    import threading
    import gpubridge_b200 as gb

    class Recorder(gb.CollectiveObserver):
        def __init__(self):
            self.records, self.detached = [], None

        def on_collective(self, record):
            self.records.append(record)

        def on_detach(self, error):
            self.detached = error

    class Chatty(Recorder):
        def on_collective(self, record):
            gb.barrier()                       # observers must not communicate

    with pytest.raises(TypeError):
        gb.add_observer(object())
    rec = Recorder()
    gb.add_observer(rec)
    gb.add_observer(rec)                       # idempotent
    t = rank_tensor(rank, 100)
    gb.all_reduce(t, gb.ReduceOp.AVG)
    gb.broadcast(t, 3)
    gb.barrier()
    ops = [(r.seq, r.op, r.reduce_op, r.src) for r in rec.records]
    assert ops == [(0, "all_reduce", "avg", None), (1, "broadcast", None, 3), (2, "barrier", None, None)]
    first = rec.records[0]
    assert first.policy == "reduce-bridge-broadcast" and first.nbytes == 400 and first.ready()
    names = [p.name for p in first.phases]
    assert names == (["island-reduce", "bridge", "island-broadcast"] if topology.is_leader
                     else ["island-reduce", "island-broadcast"])
    assert first.elapsed_ms() >= 0 and first.phase("island-reduce").elapsed_ms() >= 0
    assert first.phase("nope") is None and rec.records[2].nbytes == 0
    # a failing observer is detached with a warning; collectives carry on
    bad = Chatty()
    gb.add_observer(bad)
    with pytest.warns(RuntimeWarning, match="detached collective observer"):
        gb.all_reduce(t)
    assert isinstance(bad.detached, RuntimeError) and "must not communicate" in str(bad.detached)
    gb.all_reduce(t)
    gb.remove_observer(rec)
    before = len(rec.records)
    gb.all_reduce(t)
    assert len(rec.records) == before
    # in_flight: visible from another thread while a collective runs on this one
    assert gb.in_flight() == []
    seen = []
    stop = threading.Event()

    def watch():
        while not stop.is_set():
            seen.extend(gb.in_flight())

    watcher = threading.Thread(target=watch)
    watcher.start()
    for _ in range(20):
        gb.all_reduce(rank_tensor(rank, 50_000))
    stop.set()
    watcher.join()
    assert all(f.op == "all_reduce" and f.seconds >= 0 for f in seen)
    assert {f.phase for f in seen} <= {None, "island-reduce", "bridge", "island-broadcast"}
    return len(seen)


def test_observers_and_in_flight(tmp_path):
    run_ranks(TWO_BY_TWO, _observe, tmp_path)


def _queue(rank, topology):
    import gpubridge_b200 as gb
    from gpubridge_b200 import work
    world = topology.world_size
    # FIFO: async collectives complete in submission order, a blocking call drains them first
    works = [gb.all_reduce(rank_tensor(rank, 10 + i), async_op=True) for i in range(3)]
    t = rank_tensor(rank, 5)
    gb.all_reduce(t)
    assert all(w.is_completed() for w in works)
    assert torch.equal(t, expected_sum(world, 5))
    with pytest.raises(TimeoutError):
        class Never(work.Work):
            pass
        Never("x", topology.device, None).wait(0.01)
    # the queue is bounded: overflow rejects the new call, accepted work keeps its order
    held = [gb.all_reduce(rank_tensor(rank, 200_000), async_op=True) for _ in range(2)]
    extra = []
    try:
        for _ in range(50):
            extra.append(gb.all_reduce(rank_tensor(rank, 3), async_op=True))
    except RuntimeError as exc:
        assert "queue is full" in str(exc)
    for w in held + extra:
        w.wait()
    return len(extra)


def test_async_queue_is_fifo_and_bounded(tmp_path):
    # every rank must hit the limit at the same call for the sequence to stay aligned: a queue
    # of 64 is never full here, so no rank rejects and all 50 extra calls go through
    counts = run_ranks(TWO_BY_TWO, _queue, tmp_path, env={"GPUBRIDGE_ASYNC_QUEUE": "64"})
    assert counts == [50] * 4


def _poison(rank, topology):
    import gpubridge_b200 as gb
    from gpubridge_b200 import policies

    class Boom(policies.FlatGloo):
        name = "boom"

        def all_reduce(self, tensor, topology, op="sum"):
            raise OSError("link down")

    broken = Boom()
    object.__setattr__(topology, "policy", broken)
    w = gb.all_reduce(torch.ones(4), async_op=True)
    with pytest.raises(RuntimeError, match="link down"):
        w.wait()
    assert isinstance(w.exception(), OSError)
    with pytest.raises(RuntimeError, match="earlier async gpubridge collective failed"):
        gb.all_reduce(torch.ones(4))
    with pytest.raises(RuntimeError, match="earlier async gpubridge collective failed"):
        gb.barrier(async_op=True)
    return True


def test_first_async_failure_poisons_the_rank(tmp_path):
    run_ranks(TWO_BY_TWO, _poison, tmp_path)


def _reinit(rank, world, path):
    from datetime import timedelta
    import gpubridge_b200 as gb
    for generation in range(2):
        topology = gb.init(f"file://{path}.{generation}", rank=rank, world_size=world,
                           timeout=timedelta(seconds=30))
        with pytest.raises(RuntimeError, match="already initialized"):
            gb.init(f"file://{path}.x", rank=rank, world_size=world)
        t = rank_tensor(rank, 9)
        gb.all_reduce(t)
        assert torch.equal(t, expected_sum(world, 9))
        assert gb.is_initialized() and gb.get_topology() is topology
        gb.destroy()
        gb.destroy()                               # a second destroy does nothing
        assert not gb.is_initialized()
        with pytest.raises(RuntimeError, match="not initialized"):
            gb.all_reduce(t)
    return True


def test_destroy_and_init_again(tmp_path):
    run_ranks(TWO_BY_TWO, _reinit, tmp_path, mode="raw")


def test_marks_that_arrive_later():
    """Device timestamps of a fused kernel reach the host by an asynchronous copy: the phases
    exist at once, are ready when the copy's event is, and read the pinned buffer lazily."""
    import torch
    from gpubridge_b200 import observe

    class Event:
        def __init__(self): self.done = False
        def query(self): return self.done

    stamps = torch.zeros(3, dtype=torch.int64)
    event = Event()
    flight = observe._Flight(1, "all_reduce", "p")
    flight.watched = True
    observe._local.flight = flight
    try:
        observe.device_phases_later(["island-reduce", "bridge-reduce"], stamps, event)
    finally:
        observe._local.flight = None
    assert [p.name for p in flight.phases] == ["island-reduce", "bridge-reduce"]
    assert flight.done == ("island-reduce", "bridge-reduce")
    assert not flight.phases[0].start.ready()
    stamps.copy_(torch.tensor([1_000_000, 3_500_000, 4_000_000]))      # the copy lands
    event.done = True
    assert flight.phases[0].end.ready()
    assert flight.phases[0].elapsed_ms() == 2.5 and flight.phases[1].elapsed_ms() == 0.5
    assert observe.Mark(0, None, 7).ns() == 7 and observe.Mark(0).ns() is None


def _nvtx_ranges(rank, topology):
    import gpubridge_b200 as gb
    from gpubridge_b200 import observe

    class Recorder:
        def __init__(self):
            self.events, self.depth = [], 0

        def range_push(self, name):
            self.depth += 1
            self.events.append(("push", name, self.depth))

        def range_pop(self):
            self.events.append(("pop", None, self.depth))
            self.depth -= 1

    recorder = observe._nvtx = Recorder()
    try:
        gb.all_reduce(torch.ones(10))
        gb.broadcast(torch.ones(4), 0)
    finally:
        observe._nvtx = None
    return recorder.events, recorder.depth


def test_nvtx_ranges_bracket_collectives_and_phases(tmp_path):
    events, depth = run_ranks(("nvidia", "amd"), _nvtx_ranges, tmp_path)[0]
    assert depth == 0 and len([e for e in events if e[0] == "push"]) == len([e for e in events if e[0] == "pop"])
    names = [name for kind, name, _ in events if kind == "push"]
    assert names[0] == "gpubridge.all_reduce 40" and "gpubridge.broadcast 16" in names
    inner = [name for kind, name, level in events if kind == "push" and level == 2]
    assert "gpubridge.bridge" in inner           # phases nest inside their collective
