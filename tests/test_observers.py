"""Collective observers and ``in_flight`` beyond the happy path: sequence numbers are the
collective's position in the job, the same on every rank whenever an observer was attached;
a refused call uses none; an observer that raises is detached where it raised and nowhere
else; nothing can be attached or seen before ``init``; a collective that failed is forgotten;
phases nest.  (Reference: tests/test_observe.py.)"""
import pytest
import torch

from _harness import TWO_BY_TWO, rank_tensor, run_ranks


def test_nothing_to_observe_before_init():
    import gpubridge_b200 as gb

    class Quiet(gb.CollectiveObserver):
        def on_collective(self, record):
            pass

    assert gb.in_flight() == []
    with pytest.raises(RuntimeError):
        gb.add_observer(Quiet())
    gb.remove_observer(Quiet())                                    # removing what was never there is not an error
    with pytest.raises(TypeError):
        gb.CollectiveObserver()                                    # abstract


def _late_attach(rank, topology):
    import gpubridge_b200 as gb

    class Recorder(gb.CollectiveObserver):
        def __init__(self):
            self.records = []

        def on_collective(self, record):
            self.records.append(record)

    rec = Recorder()
    t = rank_tensor(rank, 64)
    # ranks attach after a different number of collectives: numbers still name the same call everywhere
    for i in range(4):
        if i == rank:
            gb.add_observer(rec)
        gb.all_reduce(t.clone())
    gb.broadcast(t, 0)
    return [(r.seq, r.op, r.nbytes, str(r.dtype), r.policy) for r in rec.records]


def test_sequence_numbers_match_even_when_ranks_attach_at_different_times(tmp_path):
    out = run_ranks(TWO_BY_TWO, _late_attach, tmp_path)
    for rank, records in enumerate(out):
        assert [seq for seq, *_ in records] == list(range(rank, 5))
    by_seq = {}
    for records in out:
        for seq, *rest in records:
            by_seq.setdefault(seq, set()).add(tuple(rest))
    assert all(len(v) == 1 for v in by_seq.values())               # every rank describes call n alike
    assert by_seq[4] == {("broadcast", 256, "torch.float32", "reduce-bridge-broadcast")}


def _refused(rank, topology):
    import gpubridge_b200 as gb

    class Recorder(gb.CollectiveObserver):
        def __init__(self):
            self.seqs = []

        def on_collective(self, record):
            self.seqs.append((record.seq, record.op))

    rec = Recorder()
    gb.add_observer(rec)
    gb.all_reduce(rank_tensor(rank, 8))
    for bad in (lambda: gb.all_reduce(torch.ones(4).to_sparse()), lambda: gb.broadcast(torch.ones(4), 99),
                lambda: gb.all_reduce(torch.ones(2, 4).t()), lambda: gb.all_reduce("not a tensor")):
        with pytest.raises((ValueError, TypeError, RuntimeError)):
            bad()
    assert gb.in_flight() == []                                    # a refused call was never in flight
    gb.all_reduce(rank_tensor(rank, 8))
    return rec.seqs


def test_rejected_calls_do_not_use_a_sequence_number(tmp_path):
    out = run_ranks(TWO_BY_TWO, _refused, tmp_path)
    assert all(seqs == [(0, "all_reduce"), (1, "all_reduce")] for seqs in out)


def _one_rank_raises(rank, topology):
    import warnings

    import gpubridge_b200 as gb

    class Fragile(gb.CollectiveObserver):
        def __init__(self):
            self.seen, self.detached = 0, None

        def on_collective(self, record):
            self.seen += 1
            if rank == 1 and self.seen == 2:
                raise KeyError("my own bug")

        def on_detach(self, error):
            self.detached = repr(error)
            raise RuntimeError("and the detach hook is broken too")       # must not matter either

    obs = Fragile()
    gb.add_observer(obs)
    caught = []
    for _ in range(4):
        with warnings.catch_warnings(record=True) as seen:
            warnings.simplefilter("always")
            gb.all_reduce(rank_tensor(rank, 16))
        caught += [str(w.message) for w in seen if issubclass(w.category, RuntimeWarning)]
    return obs.seen, obs.detached, caught


def test_an_observer_that_raises_is_detached_on_its_rank_only(tmp_path):
    out = run_ranks(TWO_BY_TWO, _one_rank_raises, tmp_path)
    for rank, (seen, detached, warned) in enumerate(out):
        if rank == 1:
            assert seen == 2 and "my own bug" in detached
            assert len(warned) == 1 and "detached collective observer" in warned[0] and "KeyError" in warned[0]
        else:
            assert seen == 4 and detached is None and warned == []


def _nested_and_failed(rank, topology):
    import gpubridge_b200 as gb
    from gpubridge_b200 import observe

    class Recorder(gb.CollectiveObserver):
        def __init__(self):
            self.records = []

        def on_collective(self, record):
            self.records.append(record)

    rec = Recorder()
    gb.add_observer(rec)
    snapshots = []
    with observe.collective(topology, "all_reduce", torch.zeros(3), policy="mine"):
        with observe.phase("outer"):
            with observe.phase("inner"):
                snapshots.append(gb.in_flight()[0])
            snapshots.append(gb.in_flight()[0])
        snapshots.append(gb.in_flight()[0])
    assert [(s.phase, s.phases_done) for s in snapshots] == [
        ("inner", ()), ("outer", ("inner",)), (None, ("inner", "outer"))]
    assert snapshots[0].op == "all_reduce" and snapshots[0].policy == "mine" and snapshots[0].seconds >= 0
    record = rec.records[-1]
    assert [p.name for p in record.phases] == ["inner", "outer"] and record.nbytes == 12
    assert record.phase("outer").elapsed_ms() >= record.phase("inner").elapsed_ms() >= 0
    with observe.phase("outside any collective"):                  # a no-op, not an error
        pass
    # a collective that fails is forgotten: not in flight afterwards, no record, but its number is used
    before = len(rec.records)
    with pytest.raises(ZeroDivisionError):
        with observe.collective(topology, "broadcast", torch.zeros(3), src=0):
            with observe.phase("bridge"):
                1 / 0
    assert gb.in_flight() == [] and len(rec.records) == before
    gb.barrier()
    assert rec.records[-1].op == "barrier" and rec.records[-1].seq == record.seq + 2
    gb.remove_observer(rec)
    gb.remove_observer(rec)
    return True


def test_in_flight_tracks_nested_phases_and_forgets_failed_calls(tmp_path):
    run_ranks(TWO_BY_TWO, _nested_and_failed, tmp_path)


def _unwatched(rank, topology):
    import gpubridge_b200 as gb
    from gpubridge_b200 import observe
    assert not observe.watching()
    made = []
    original = observe._mark
    observe._mark = lambda device: made.append(device) or original(device)
    try:
        for _ in range(3):
            gb.all_reduce(rank_tensor(rank, 32))
    finally:
        observe._mark = original
    return len(made)


def test_without_an_observer_no_call_is_timed(tmp_path):
    assert run_ranks(TWO_BY_TWO, _unwatched, tmp_path) == [0, 0, 0, 0]
