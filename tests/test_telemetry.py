"""The JSON-lines emitter: records arrive in order with the run's constant fields, a full queue
drops and counts instead of blocking, names that look like secrets are refused, the file only
takes its name when the run closed it, and collectives can be recorded through an observer."""
import json
import os
import time

import pytest
import torch

from gpubridge_b200 import telemetry


def read(path):
    with open(path) as fh:
        return [json.loads(line) for line in fh]


def test_records_arrive_in_order_with_the_constant_fields(tmp_path):
    path = tmp_path / "run" / "obs.jsonl"
    with telemetry.Emitter(path, run="unit", rank=3) as emitter:
        for i in range(50):
            assert emitter.emit("step", index=i, ms=0.5 * i, tags=["a", "b"], nested={"x": 1})
        assert not os.path.exists(path) and os.path.exists(str(path) + ".partial")
    rows = read(path)
    assert [r["index"] for r in rows[:-1]] == list(range(50))
    assert all(r["run"] == "unit" and r["rank"] == 3 and r["kind"] == "step" for r in rows[:-1])
    assert rows[-1]["kind"] == "closed" and rows[-1]["written"] == 50 and rows[-1]["dropped"] == 0
    assert not os.path.exists(str(path) + ".partial")


@pytest.mark.parametrize("name", ["rkey", "api_token", "Password", "remote_key", "aws_secret", "credentials"])
def test_names_that_look_like_secrets_are_refused(tmp_path, name):
    with telemetry.Emitter(tmp_path / "o.jsonl") as emitter:
        with pytest.raises(ValueError, match="credential or a memory key"):
            emitter.emit("x", **{name: 1})
        with pytest.raises(ValueError):
            emitter.emit("x", outer={name: 1})
    with pytest.raises(ValueError):
        telemetry.Emitter(tmp_path / "p.jsonl", **{name: "v"})


def test_only_json_values_travel(tmp_path):
    with telemetry.Emitter(tmp_path / "o.jsonl") as emitter:
        with pytest.raises(ValueError, match="Tensor"):
            emitter.emit("x", value=torch.ones(1))
        assert emitter.emit("x", value=1.5, names=("a", "b"), maybe=None)


def test_a_full_queue_drops_and_counts_without_blocking(tmp_path):
    emitter = telemetry.Emitter(tmp_path / "o.jsonl", capacity=4)
    emitter._queue.put({"kind": "stall"})                     # keep the writer busy with a blocker below

    class Slow(dict):
        pass

    began = time.monotonic()
    sent = [emitter.emit("burst", index=i) for i in range(5000)]
    assert time.monotonic() - began < 2.0
    emitter.close()
    rows = read(tmp_path / "o.jsonl")
    closing = rows[-1]
    assert closing["kind"] == "closed" and closing["dropped"] == sent.count(False)
    assert closing["written"] + closing["dropped"] >= 5000
    if closing["dropped"]:
        assert any("dropped_before" in r for r in rows) or closing["dropped"] > 0
    assert emitter.emit("late") is False


def test_an_endpoints_counters_become_a_record(tmp_path):
    from gpubridge_b200 import rdma
    from gpubridge_b200.ops import _lib
    if not _lib.available():
        pytest.skip("the native library is not built")
    fabric = rdma.MockFabric(2)
    try:
        a = fabric.endpoint(0)
        fabric.endpoint(1)
        with telemetry.Emitter(tmp_path / "e.jsonl", rank=0) as emitter:
            assert emitter.endpoint(a)
        row = read(tmp_path / "e.jsonl")[0]
        assert row["kind"] == "endpoint" and row["member"] == 0 and row["eager_sent"] == 0
    finally:
        fabric.close()


def test_collectives_are_recorded_through_an_observer(tmp_path):
    """The observer turns a record into a line (observers can only be attached to an
    initialised job, so the record is handed over directly here)."""
    from gpubridge_b200 import observe
    mark = observe.Mark(time.perf_counter_ns())
    later = observe.Mark(mark.host_ns + 2_000_000)
    record = observe.CollectiveRecord(seq=4, op="all_reduce", nbytes=64, dtype=torch.float32, src=None,
                                      policy="native-only", start=mark, end=later,
                                      phases=(observe.Phase("island-reduce", mark, later),), reduce_op="sum")
    with telemetry.Emitter(tmp_path / "c.jsonl", rank=0) as emitter:
        telemetry.CollectiveEmitter(emitter).on_collective(record)
    row = read(tmp_path / "c.jsonl")[0]
    assert row["op"] == "all_reduce" and row["nbytes"] == 64 and row["policy"] == "native-only"
    assert row["phases"] == {"island-reduce": 2.0} and row["ms"] == 2.0 and row["seq"] == 4
