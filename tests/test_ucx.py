"""``bridge="ucx"``: the worker of ``ucx/gb_ucx.cpp`` compiled against the stand-in UCP library of
``tests/fake_ucx`` (same API, Unix-domain sockets underneath), which lets tests make UCX
misbehave: members in threads for the worker itself, ranks in processes for the bridge of the
policies and for what init promises when one leader's UCX is different or does not start.
What needs no UCX at all (tags, cuts, settings, the path table, the refusal without UCX) runs
first."""
import json
import os
import subprocess
import sys
import threading
import time
from datetime import timedelta

import pytest
import torch

import _fake_ucx
from _harness import LAYOUTS, expected_sum, rank_tensor, run_ranks
from gpubridge_b200 import tagged, transport

HAVE_COMPILER = _fake_ucx.shutil.which("c++") or _fake_ucx.shutil.which("g++")
needs_compiler = pytest.mark.skipif(not HAVE_COMPILER, reason="no C++ compiler")


# ---- without any UCX ---------------------------------------------------------------------------------
def test_tags_keep_call_step_sender_and_chunk_apart():
    seen = {tagged.message_tag(n, s, m, c) for n in (1, 2, 0xFFFFFF) for s in (0, 1, 0xFFF)
            for m in (0, 1, 255) for c in (0, 1, 0xFFFFF)}
    assert len(seen) == 81 and max(seen) < 1 << 64
    assert tagged.message_tag(1 << 24, 0, 0, 0) == tagged.message_tag(0, 0, 0, 0)       # the call number wraps


@pytest.mark.parametrize("numel, parts", [(10, 3), (2, 4), (0, 2), (1000, 8), (7, 7)])
def test_segments_cover_the_tensor_once(numel, parts):
    cuts = tagged.segments(numel, parts)
    assert len(cuts) == parts and cuts[0][0] == 0 and sum(n for _, n in cuts) == numel
    assert all(a[0] + a[1] == b[0] for a, b in zip(cuts, cuts[1:]))
    assert max(n for _, n in cuts) - min(n for _, n in cuts) <= 1 and cuts[0][1] == max(n for _, n in cuts)


def test_chunk_size_setting(monkeypatch):
    from gpubridge_b200.ucx import transport as ut
    monkeypatch.delenv(ut.CHUNK_ENV, raising=False)
    assert ut.chunk_bytes_setting() == 4 << 20
    monkeypatch.setenv(ut.CHUNK_ENV, "64K")
    assert ut.chunk_bytes_setting() == 65536
    for bad in ("7", "0", "lots"):
        monkeypatch.setenv(ut.CHUNK_ENV, bad)
        with pytest.raises(ValueError, match=ut.CHUNK_ENV):
            ut.chunk_bytes_setting()


@pytest.mark.parametrize("device, contiguous, types, direct_ok, want", [
    ("cpu", True, {"host"}, True, "host"), ("cpu", False, {"host"}, True, "staged"),
    ("cuda", True, {"host"}, True, "staged"), ("cuda", True, {"host", "cuda"}, True, "direct"),
    ("cuda", True, {"host", "cuda"}, False, "staged"), ("cuda", False, {"host", "cuda"}, True, "staged")])
def test_device_tensors_go_direct_only_where_ucx_has_their_memory(device, contiguous, types, direct_ok, want):
    from gpubridge_b200.ucx import transport as ut
    assert ut.choose_path(device, contiguous, types, direct_ok) == want


def test_without_ucx_the_bridge_says_why(monkeypatch, tmp_path):
    from gpubridge_b200 import ucx
    monkeypatch.delenv("UCX_HOME", raising=False)
    monkeypatch.setenv("PATH", str(tmp_path))                  # no pkg-config either
    if os.path.exists("/usr/include/ucp/api/ucp.h"):
        pytest.skip("this machine has UCX")
    with pytest.raises(ValueError, match="can't be loaded.*UCX was not found"):
        transport.resolve_transport("ucx")
    with pytest.raises(ucx.Unavailable, match="UCX was not found"):
        ucx.ucx_flags()
    assert ucx.info()["found"] is False
    monkeypatch.setenv("UCX_HOME", str(tmp_path))
    with pytest.raises(ucx.Unavailable, match="has no include/ucp/api/ucp.h"):
        ucx.ucx_flags()


def test_the_command_line_without_ucx():
    if os.path.exists("/usr/include/ucp/api/ucp.h"):
        pytest.skip("this machine has UCX")
    env = {k: v for k, v in os.environ.items() if k != "UCX_HOME"}
    done = subprocess.run([sys.executable, "-m", "gpubridge_b200.ucx", "info"], capture_output=True, text=True, env=env)
    assert json.loads(done.stdout)["found"] is False
    done = subprocess.run([sys.executable, "-m", "gpubridge_b200.ucx", "build"], capture_output=True, text=True, env=env)
    assert done.returncode == 1 and "nothing built" in done.stderr
    done = subprocess.run([sys.executable, "-m", "gpubridge_b200.ucx", "polish"], capture_output=True, text=True, env=env)
    assert done.returncode == 2


# ---- with the stand-in UCX ---------------------------------------------------------------------------
@pytest.fixture(scope="module")
def fake_ucx(tmp_path_factory):
    if not HAVE_COMPILER:
        pytest.skip("no C++ compiler")
    prefix = _fake_ucx.install(tmp_path_factory.mktemp("ucx-prefix"))
    settings = {"UCX_HOME": str(prefix), "GPUBRIDGE_UCX_LIB_DIR": str(prefix / "cache")}
    before = {k: os.environ.get(k) for k in settings}
    os.environ.update(settings)
    from gpubridge_b200 import ucx
    ucx.build()
    yield settings
    for key, value in before.items():
        if value is None:
            os.environ.pop(key, None)
        else:
            os.environ[key] = value


def _workers(count, body, leave_together=True):
    """``body(worker, index)`` on ``count`` connected workers, one thread each."""
    from gpubridge_b200 import ucx
    addresses, ready, finished = [None] * count, threading.Barrier(count), threading.Barrier(count)
    out, errors = [None] * count, []

    def run(i):
        worker = None
        try:
            worker = ucx.Worker(count, i)
            addresses[i] = worker.address()
            ready.wait(20)
            for j in range(count):
                if j != i:
                    worker.connect(j, addresses[j])
            out[i] = body(worker, i)
            if leave_together:
                finished.wait(30)
        except BaseException as failure:  # noqa: BLE001
            errors.append((i, repr(failure)))
            finished.abort()
        finally:
            if worker is not None:
                worker.close(5.0)

    threads = [threading.Thread(target=run, args=(i,)) for i in range(count)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(60)
    assert not errors, errors
    return out


def test_the_worker_is_built_per_ucx_and_reports_its_version(fake_ucx, tmp_path, monkeypatch):
    from gpubridge_b200 import ucx
    assert ucx.version() == (1, 17, 0)
    first = ucx.library_path()
    assert first.exists() and first.parent == _fake_ucx.Path(fake_ucx["GPUBRIDGE_UCX_LIB_DIR"])
    told = ucx.info()
    assert told["found"] and told["built"] and told["library"] == str(first)
    # another UCX at another prefix (a different version header): another library name
    other = tmp_path / "other"
    _fake_ucx.shutil.copytree(fake_ucx["UCX_HOME"], other)
    header = other / "include" / "ucp" / "api" / "ucp_version.h"
    header.write_text(header.read_text().replace("UCP_API_MINOR 17", "UCP_API_MINOR 18"))
    monkeypatch.setenv("UCX_HOME", str(other))
    assert ucx.library_path() != first and not ucx.library_path().exists()


@pytest.mark.parametrize("count", [2, 3, 4])
def test_native_collectives_over_the_worker(fake_ucx, count):
    def body(worker, i):
        deadline = time.monotonic() + 30
        assert worker.memory_types() == {"host"}
        outs = []
        for dtype, code in ((torch.float32, 0), (torch.int64, 7), (torch.bfloat16, 1)):
            t = rank_tensor(i, 300_001, dtype)
            worker.all_reduce(t.data_ptr(), t.numel(), code, 0, 50_000, len(outs) + 1, deadline)
            outs.append(t)
        b = torch.full((70_000,), float(i))
        worker.broadcast(b.data_ptr(), b.nbytes, count - 1, 1 << 16, 9, deadline)
        return outs, b, worker.telemetry()

    for outs, b, counters in _workers(count, body):
        for t, dtype in zip(outs, (torch.float32, torch.int64, torch.bfloat16)):
            assert torch.equal(t, expected_sum(count, 300_001, dtype))
        assert torch.equal(b, torch.full((70_000,), float(count - 1)))
        assert counters["open_operations"] == 0 and not counters["broken"] and counters["sends"] > 0


@pytest.mark.parametrize("count, op", [(2, "sum"), (3, "sum"), (4, "max"), (3, "min")])
def test_message_by_message_collectives_give_the_native_bits(fake_ucx, count, op):
    """``OnDevice`` (used where the reduction has to run on a device) cuts, orders and tags like
    the native code: floating-point sums come out bit for bit the same."""
    torch.manual_seed(5)
    values = [torch.randn(100_003) * 10 ** (i - 1) for i in range(count)]

    def body(worker, i):
        deadline = time.monotonic() + 30
        native, stepwise = values[i].clone(), values[i].clone()
        worker.all_reduce(native.data_ptr(), native.numel(), 0, tagged.OP_CODES[op], 7_000, 1, deadline)
        calls = []
        walker = tagged.OnDevice(worker, count, i, settle=lambda: calls.append("settle"),
                                 landed=lambda: calls.append("landed"))
        walker.all_reduce(stepwise, op, 7_000, 2, deadline)
        sent = torch.full((999,), float(i))
        walker.broadcast(sent, 1, 512, 3, deadline)
        return native, stepwise, sent, calls

    out = _workers(count, body)
    for i, (native, stepwise, sent, calls) in enumerate(out):
        assert torch.equal(native, stepwise) and torch.equal(native, out[0][0])
        assert torch.equal(sent, torch.full((999,), 1.0))
        assert calls[0] == "settle" and "landed" in calls
        assert calls.index("landed") > calls.index("settle")


@pytest.mark.parametrize("count", [2, 3])
def test_native_and_message_by_message_members_understand_each_other(fake_ucx, count):
    """Same tags, cuts and steps on both sides: member 0 runs the native code, the others walk
    the messages from Python, inside one and the same call."""
    def body(worker, i):
        deadline = time.monotonic() + 30
        t = rank_tensor(i, 50_001)
        if i == 0:
            worker.all_reduce(t.data_ptr(), t.numel(), 0, 0, 3_000, 1, deadline)
        else:
            tagged.OnDevice(worker, count, i).all_reduce(t, "sum", 3_000, 1, deadline)
        return t

    for t in _workers(count, body):
        assert torch.equal(t, expected_sum(count, 50_001))


def test_a_message_shorter_than_its_receive_is_an_error_not_garbage(fake_ucx):
    from gpubridge_b200 import ucx

    def body(worker, i):
        deadline = time.monotonic() + 10
        if i == 0:
            short = torch.ones(25)
            worker.wait([worker.send(1, short.data_ptr(), short.nbytes, 4)], deadline)
            return None
        room = torch.zeros(50)
        with pytest.raises(ucx.UcxError, match="25|100") as caught:
            worker.wait([worker.recv(0, room.data_ptr(), room.nbytes, 4)], deadline)
        assert "disagree" in str(caught.value)
        with pytest.raises(ucx.UcxError, match="disagree"):              # broken for good, first reason kept
            worker.recv(0, room.data_ptr(), room.nbytes, 5)
        return worker.telemetry()["broken"]

    assert _workers(2, body)[1] == 1


def test_a_message_longer_than_its_receive_is_ucxs_truncation_error(fake_ucx):
    from gpubridge_b200 import ucx

    def body(worker, i):
        deadline = time.monotonic() + 10
        if i == 0:
            long = torch.ones(50)
            worker.wait([worker.send(1, long.data_ptr(), long.nbytes, 4)], deadline)
            return None
        room = torch.zeros(25)
        with pytest.raises(ucx.UcxError, match="[Tt]runcated"):
            worker.wait([worker.recv(0, room.data_ptr(), room.nbytes, 4)], deadline)
        return True

    assert _workers(2, body)[1]


def test_messages_that_arrive_before_their_receive_are_kept(fake_ucx):
    def body(worker, i):
        deadline = time.monotonic() + 10
        if i == 0:
            payloads = [torch.full((3000,), float(k)) for k in range(20)]
            worker.wait([worker.send(1, p.data_ptr(), p.nbytes, 100 + k) for k, p in enumerate(payloads)], deadline)
            return None
        time.sleep(0.3)                                          # the sender is done before anything is posted
        outs = [torch.zeros(3000) for _ in range(20)]
        order = list(reversed(range(20)))                        # and the receives come in another order
        worker.wait([worker.recv(0, outs[k].data_ptr(), outs[k].nbytes, 100 + k) for k in order], deadline)
        return [float(o[0]) for o in outs]

    assert _workers(2, body)[1] == [float(k) for k in range(20)]


def test_a_receive_nobody_answers_trips_the_deadline_and_breaks_the_worker(fake_ucx):
    from gpubridge_b200 import ucx

    def body(worker, i):
        if i == 0:
            return None
        room = torch.zeros(10)
        started = time.monotonic()
        with pytest.raises(ucx.UcxError, match="timed out") as caught:
            worker.wait([worker.recv(0, room.data_ptr(), room.nbytes, 1)], time.monotonic() + 0.5)
        assert caught.value.code == ucx.TIMED_OUT and time.monotonic() - started < 5
        with pytest.raises(ucx.UcxError, match="deadline"):
            worker.all_reduce(room.data_ptr(), 10, 0, 0, 10, 2, time.monotonic() + 1)
        counters = worker.telemetry()
        return counters["broken"], counters["open_operations"]

    assert _workers(2, body)[1] == (1, 0)                        # the receive was cancelled and collected


def test_closing_with_an_operation_outstanding_returns_in_time(fake_ucx):
    def body(worker, i):
        room = torch.zeros(1 << 20)
        worker.recv(1 - i, room.data_ptr(), room.nbytes, 77)     # never matched, never waited for
        return room                                              # stays alive past close

    started = time.monotonic()
    _workers(2, body)
    assert time.monotonic() - started < 20


def test_sending_to_a_member_that_is_not_connected_is_refused_not_fatal(fake_ucx):
    from gpubridge_b200 import ucx
    worker = ucx.Worker(2, 0)
    try:
        t = torch.zeros(4)
        with pytest.raises(ucx.UcxError, match="not connected"):
            worker.send(1, t.data_ptr(), t.nbytes, 1)
        with pytest.raises(ucx.UcxError, match="not connected"):
            worker.send(0, t.data_ptr(), t.nbytes, 1)            # itself
        assert worker.telemetry()["broken"] == 0
        with pytest.raises(ucx.UcxError, match="no such member"):
            worker.connect(5, b"x" * 104)
        with pytest.raises(ucx.UcxError, match="ucp_ep_create"):
            worker.connect(1, b"not an address" + bytes(90))
    finally:
        worker.close(1.0)
    with pytest.raises(ucx.UcxError, match="closed"):
        worker.telemetry()


def test_ucx_that_does_not_start_is_reported_with_advice(fake_ucx, monkeypatch):
    from gpubridge_b200 import ucx
    monkeypatch.setenv("FAKE_UCP_FAIL_INIT", "1")
    with pytest.raises(ucx.UcxError, match="No such device.*UCX_TLS"):
        ucx.Worker(2, 0)
    with pytest.raises(ucx.UcxError, match="member count or index"):
        ucx.Worker(2, 2)


def _transports(count, body, chunk=1 << 16, **settings):
    from gpubridge_b200.ucx.transport import UcxTransport

    def wrapped(worker, i):
        bridge = UcxTransport(worker, list(range(10, 10 + count)), 10 + i, timedelta(seconds=20), chunk, **settings)
        try:
            return body(bridge, i)
        finally:
            bridge.worker = None                                 # the thread helper closes the worker
    return _workers(count, wrapped)


@pytest.mark.parametrize("count", [2, 3])
def test_the_three_paths_of_the_transport(fake_ucx, count):
    from gpubridge_b200.rdma_transport import Route, Router

    class EverythingInPlace(Router):
        def _route(self, tensor):
            return Route("in-place", "the test says so") if tensor.is_contiguous() else super()._route(tensor)

    def body(bridge, i):
        seen = []
        host = rank_tensor(i, 40_001)
        bridge.all_reduce(host)
        seen.append(bridge.last_path)
        strided = rank_tensor(i, 40_000).view(200, 200).t()
        bridge.all_reduce(strided)
        seen.append(bridge.last_path)
        counted = bridge.router.counts
        bridge.router = EverythingInPlace()
        bridge.router.counts = counted
        direct = rank_tensor(i, 40_001)
        bridge.all_reduce(direct, "max")
        seen.append(bridge.last_path)
        sent = torch.full((5000,), float(i))
        bridge.broadcast(sent, 11)
        return host, strided, direct, sent, seen, bridge.describe()

    for host, strided, direct, sent, seen, told in _transports(count, body, piece_bytes=32 << 10):
        assert seen == ["host", "staged", "direct"]
        assert torch.equal(host, expected_sum(count, 40_001))
        assert torch.equal(strided, expected_sum(count, 40_000).view(200, 200).t())
        assert torch.equal(direct, torch.stack([rank_tensor(r, 40_001) for r in range(count)]).max(0).values)
        assert torch.equal(sent, torch.full((5000,), 1.0))
        assert told["paths"]["staged"] == 1 and told["staging"]["allocated"] == 1
        assert told["endpoint"]["open_operations"] == 0


def test_a_failed_call_stops_the_worker_before_the_caller_sees_it(fake_ucx):
    from gpubridge_b200 import ucx

    def body(bridge, i):
        bridge.timeout = 0.5
        if i == 0:
            return None                                          # never joins the call
        with pytest.raises(ucx.UcxError, match="timed out"):
            bridge.all_reduce(torch.ones(1000))
        with pytest.raises(ucx.UcxError):
            bridge.all_reduce(torch.ones(10))
        return bridge.worker.telemetry()["broken"]

    assert _transports(2, body)[1] == 1


# ---- between processes -------------------------------------------------------------------------------
def _through_ucx(rank, topology, policy):
    import gpubridge_b200 as gb
    assert topology.peers[rank].bridge == "ucx"
    world = topology.world_size
    for n in (1, 1000, 300_001):
        for dtype in (torch.float32, torch.int64):
            t = rank_tensor(rank, n, dtype)
            gb.all_reduce(t)
            assert torch.equal(t, expected_sum(world, n, dtype)), (n, dtype)
    t = rank_tensor(rank, 5000)
    gb.broadcast(t, 3)
    assert torch.equal(t, rank_tensor(3, 5000))
    bridge = topology.bridge
    return topology.policy_name, None if bridge is None else bridge.last_path


@pytest.mark.parametrize("layout", ["2+2", "interleaved"])
@pytest.mark.parametrize("policy", ["auto", "pipelined-reduce-bridge-broadcast", "sharded-bridge"])
def test_every_policy_on_the_ucx_bridge_matches_the_known_sums(fake_ucx, tmp_path, layout, policy):
    out = run_ranks(LAYOUTS[layout], _through_ucx, tmp_path, policy, init={"bridge": "ucx", "policy": policy},
                    env=dict(fake_ucx, GPUBRIDGE_UCX_CHUNK_BYTES="64K"), timeout=120)
    assert len({name for name, _ in out}) == 1
    assert {path for _, path in out} <= {"host", None}


def _compressed(rank, topology):
    import gpubridge_b200 as gb
    t = (torch.arange(70_000, dtype=torch.float32) % 13 - 6) * 0.25 + rank
    want = sum((torch.arange(70_000, dtype=torch.float32) % 13 - 6) * 0.25 + r for r in range(4))
    gb.all_reduce(t)
    return float((t - want).abs().max() / want.abs().max())


@pytest.mark.parametrize("mode, bound", [("bf16", 0.02), ("fp8", 0.2)])
def test_bridge_compression_on_the_ucx_bridge(fake_ucx, tmp_path, mode, bound):
    out = run_ranks(LAYOUTS["2+2"], _compressed, tmp_path, init={"bridge": "ucx"},
                    env=dict(fake_ucx, GPUBRIDGE_BRIDGE_COMPRESSION=mode), timeout=120)
    assert max(out) < bound and len(set(out)) == 1


def _init_with(rank, world, path, per_rank, init):
    """``gb.init`` after this rank's own environment changes (what ``run_ranks`` cannot give)."""
    import warnings

    import gpubridge_b200 as gb
    os.environ.update(per_rank.get(rank, {}))
    with warnings.catch_warnings():
        warnings.simplefilter("ignore", gb.SplitTestWarning)
        started = time.monotonic()
        try:
            gb.init(f"file://{path}", rank=rank, world_size=world, timeout=timedelta(seconds=init.pop("seconds", 40)),
                    **init)
        finally:
            took = time.monotonic() - started
            if took > 30:
                raise RuntimeError(f"init took {took:.0f} s")
        gb.destroy()
    return "up"


@pytest.mark.parametrize("what, per_rank, message", [
    ("does not start", {2: {"FAKE_UCP_FAIL_INIT": "1"}}, "No such device"),
    ("another version", {0: {"FAKE_UCP_VERSION": "1.15.0"}}, "different UCX versions"),
    ("another chunk size", {2: {"GPUBRIDGE_UCX_CHUNK_BYTES": "1M"}}, "GPUBRIDGE_UCX_CHUNK_BYTES differs"),
    ("a bad setting", {0: {"GPUBRIDGE_UCX_CHUNK_BYTES": "7"}}, "multiple of 8"),
])
def test_one_leaders_trouble_fails_init_on_every_rank(fake_ucx, tmp_path, what, per_rank, message):
    errors = run_ranks(LAYOUTS["2+2"], _init_with, tmp_path, per_rank, {"bridge": "ucx"}, mode="plain",
                       env=fake_ucx, expect_error=message, timeout=90)
    assert len(errors) == 4 and all("could not be set up" in e for e in errors)


def test_leaders_that_agree_come_up(fake_ucx, tmp_path):
    same = {r: {"FAKE_UCP_VERSION": "1.15.2" if r == 0 else "1.15.0"} for r in range(4)}     # patch level may differ
    assert run_ranks(LAYOUTS["2+2"], _init_with, tmp_path, same, {"bridge": "ucx"}, mode="plain",
                     env=fake_ucx, timeout=90) == ["up"] * 4


def _leader_dies(rank, world, path):
    """Leader 2 leaves without a word after the link is up; leader 0's next call must end with
    an error well before its deadline, and say that the peer is gone."""
    import warnings

    import gpubridge_b200 as gb
    with warnings.catch_warnings():
        warnings.simplefilter("ignore", gb.SplitTestWarning)
        topology = gb.init(f"file://{path}", rank=rank, world_size=world, timeout=timedelta(seconds=25), bridge="ucx")
    t = rank_tensor(rank, 1000)
    gb.all_reduce(t)
    if rank == 2:
        os._exit(0)
    started = time.monotonic()
    try:
        gb.all_reduce(rank_tensor(rank, 100_000))
        return "no error"
    except Exception as failure:  # noqa: BLE001
        return f"{type(failure).__name__} after {time.monotonic() - started:.1f} s: {failure}"[:300]
    finally:
        del topology


def test_a_leader_that_vanishes_fails_the_other_leaders_call(fake_ucx, tmp_path):
    import multiprocessing as mp
    ctx = mp.get_context("spawn")
    results = ctx.Queue()
    path = str(tmp_path / "rdzv")
    procs = [ctx.Process(target=_vanish_entry, args=(r, path, dict(fake_ucx), results)) for r in range(4)]
    for p in procs:
        p.start()
    told = {}
    try:
        while 0 not in told:
            rank, text = results.get(timeout=80)
            told[rank] = text
    finally:
        for p in procs:
            p.join(2)
            if p.is_alive():
                p.kill()
    assert "lost a peer" in told[0] or "Connection reset" in told[0], told[0]
    seconds = float(told[0].split(" after ")[1].split(" s")[0])
    assert seconds < 15, told[0]


def _vanish_entry(rank, path, env, results):
    os.environ.update(env)
    vendors = LAYOUTS["2+2"]
    os.environ["GPUBRIDGE_VENDOR"] = vendors[rank]
    os.environ.setdefault("GPUBRIDGE_SIM_HOSTNAME", "simhost")
    torch.set_num_threads(1)
    results.put((rank, _leader_dies(rank, 4, path)))
    results.close()
    results.join_thread()                                        # the message is out before the process is
    os._exit(0)                                                  # nobody waits for a group that lost a member


# ---- point-to-point between islands over UCX ---------------------------------------------------------
def test_the_point_to_point_link_in_threads(fake_ucx):
    """Two ranks, one link each, a store that is a dict: several tags in flight at once, received
    in another order than sent, while a request that nobody answers does not keep the rest back."""
    from gpubridge_b200.ucx.p2p import UcxLink

    class Store:
        def __init__(self):
            self.items, self.ready = {}, threading.Condition()

        def set(self, key, value):
            with self.ready:
                self.items[key] = value.encode() if isinstance(value, str) else value
                self.ready.notify_all()

        def get(self, key):
            return self.items[key]

        def wait(self, keys, timeout):
            with self.ready:
                if not self.ready.wait_for(lambda: all(k in self.items for k in keys), timeout.total_seconds()):
                    raise TimeoutError(keys)

    store, out, errors = Store(), {}, []
    payloads = {tag: torch.full((50_000,), float(tag)) for tag in (3, 4, 5)}

    def run(rank):
        link = UcxLink(rank, store, timedelta(seconds=20))
        try:
            peer = 1 - rank
            if rank == 0:
                lonely = link.post(torch.zeros(8), peer, 99, False)          # never answered
                requests = [link.post(payloads[tag], peer, tag, True) for tag in (3, 4, 5)]
                for r in requests:
                    r.wait(timedelta(seconds=20))
                with pytest.raises(TimeoutError):
                    lonely.wait(timedelta(seconds=0.3))
                with pytest.raises(ValueError, match="host buffers"):
                    link.post(torch.zeros(1, device="meta"), peer, 1, True)
            else:
                rooms = {tag: torch.zeros(50_000) for tag in (5, 3, 4)}
                requests = [link.post(rooms[tag], peer, tag, False) for tag in (5, 3, 4)]
                for r in requests:
                    r.wait(timedelta(seconds=20))
                out[rank] = {tag: float(room[0]) for tag, room in rooms.items()}
        except BaseException as failure:  # noqa: BLE001
            errors.append((rank, repr(failure)))
        finally:
            link.close()
            with pytest.raises(RuntimeError, match="closed"):
                link.post(torch.zeros(1), 1 - rank, 1, True)

    threads = [threading.Thread(target=run, args=(r,)) for r in (0, 1)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(60)
    assert not errors, errors
    assert out[1] == {3: 3.0, 4: 4.0, 5: 5.0}


def _p2p_over_ucx(rank, world):
    import torch.distributed as dist
    dist.barrier()
    peer = {0: 2, 2: 0, 1: 3, 3: 1}[rank]                           # every pair crosses the islands
    lower = rank < peer
    for n in (0, 1, 4099, 300_001):
        data = (torch.arange(n) % 13).to(torch.float32) + min(rank, peer)
        if lower:
            dist.send(data, peer, tag=7)
        else:
            got = torch.full((n,), 99.0)
            dist.recv(got, peer, tag=7)
            assert torch.equal(got, data), n
    # both directions at once, batched
    mine, theirs = torch.full((10_000,), float(rank)), torch.empty(10_000)
    ops = [dist.P2POp(dist.isend, mine, peer, tag=3), dist.P2POp(dist.irecv, theirs, peer, tag=3)]
    for work in dist.batch_isend_irecv(ops):
        work.wait()
    assert float(theirs[0]) == float(peer)
    t = torch.ones(1000) * rank                                    # and the bridged collectives still work
    dist.all_reduce(t)
    assert float(t[0]) == 6.0
    from gpubridge_b200.topology import get_topology
    from gpubridge_b200.ucx.p2p import UcxLink
    backend = dist.distributed_c10d._get_default_group()
    assert get_topology().transport.name == "ucx" and isinstance(backend._engine.link, UcxLink)
    assert sorted(backend._engine.link.pairs) == [peer]
    dist.barrier()
    return True


def test_cross_island_point_to_point_over_ucx_through_the_backend(fake_ucx, tmp_path):
    run_ranks(LAYOUTS["2+2"], _p2p_over_ucx, tmp_path, mode="backend", timeout=180,
              env=dict(fake_ucx, GPUBRIDGE_BRIDGE="ucx", GPUBRIDGE_P2P_CHUNK_BYTES="64K"))


def test_the_workers_source_is_not_part_of_the_packages_own_library():
    """Everything under ``csrc/`` is compiled into the package's library on every machine; a file
    that needs UCX's headers there would break that build wherever UCX is absent."""
    from gpubridge_b200 import ucx
    from gpubridge_b200.ops import _build
    assert ucx.SOURCES[0].exists() and ucx.SOURCES[0].parent != ucx.CSRC
    for path in _build.sources():
        with open(path) as fh:
            text = fh.read()
        assert "#include <ucp/" not in text and "#include <infiniband/" not in text, path


def _three_leaders(rank, topology):
    import gpubridge_b200 as gb
    assert len(topology.layout.islands) == 3 and topology.peers[rank].bridge == "ucx"
    for n, dtype in ((300_001, torch.float32), (7, torch.int64), (50_000, torch.bfloat16)):
        t = rank_tensor(rank, n, dtype)
        gb.all_reduce(t)
        assert torch.equal(t, expected_sum(3, n, dtype)), (n, dtype)
    t = rank_tensor(rank, 999)
    gb.broadcast(t, 2)
    assert torch.equal(t, rank_tensor(2, 999))
    return topology.bridge.describe()["endpoint"]["sends"]


def test_three_leaders_run_the_workers_ring_between_processes(fake_ucx, tmp_path):
    sends = run_ranks(("nvidia",) * 3, _three_leaders, tmp_path, init={"bridge": "ucx"}, timeout=120,
                      env=dict(fake_ucx, GPUBRIDGE_ISLANDS="1,1,1", GPUBRIDGE_UCX_CHUNK_BYTES="64K"))
    assert all(count > 10 for count in sends)                      # a ring in chunks, on every leader


def test_close_from_another_thread_ends_a_blocked_wait_before_the_worker_is_freed(fake_ucx):
    from gpubridge_b200 import ucx
    seen = {}

    def body(worker, i):
        if i == 1:
            return None
        room = torch.zeros(64)

        def waits():
            try:
                worker.wait([worker.recv(1, room.data_ptr(), room.nbytes, 3)], time.monotonic() + 30)
                seen["wait"] = "returned"
            except ucx.UcxError as failure:
                seen["wait"] = str(failure)

        thread = threading.Thread(target=waits)
        thread.start()
        time.sleep(0.3)
        started = time.monotonic()
        worker.close(2.0)
        thread.join(10)
        assert not thread.is_alive() and time.monotonic() - started < 8
        with pytest.raises(ucx.UcxError, match="closed"):
            worker.memory_types()
        worker.abort()
        return seen["wait"]

    assert "UCX" in _workers(2, body)[0]


def test_the_kits_check_program_runs_over_the_ucx_bridge_and_records_its_report(fake_ucx, tmp_path):
    """The 13-stage per-rank check with ``GPUBRIDGE_BRIDGE=ucx``: every stage passes on both leaders
    and the last stage carries the bridge's own report (paths, staging, the worker's counters)."""
    out = tmp_path / "check"
    env = dict(os.environ, PYTHONPATH=os.path.dirname(os.path.dirname(os.path.abspath(__file__))), OMP_NUM_THREADS="1",
               GPUBRIDGE_VENDOR="nvidia", GPUBRIDGE_SPLIT_TEST="half", GPUBRIDGE_BRIDGE="ucx", **fake_ucx)
    done = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                           "--master-addr", "127.0.0.1", "--master-port", "29733", "-m", "gpubridge_b200.kit.check",
                           "--out", str(out), "--in-flight-settle", "0.2", "--timeout", "120"],
                          env=env, capture_output=True, text=True, timeout=300)
    assert done.returncode == 0, done.stderr[-3000:]
    for rank in (0, 1):
        record = json.loads((out / f"rank{rank}.json").read_text())
        assert record["ok"] and record["run"]["bridge"] == "ucx"
        last = record["stages"][-1]
        assert last["name"] == "destroy" and last["bridge"]["paths"].get("host", 0) > 0
        assert last["bridge"]["endpoint"]["sends"] > 0 and not last["bridge"]["endpoint"]["broken"]


@pytest.mark.parametrize("dtype, code", [(torch.bfloat16, 1), (torch.float16, 2), (torch.int64, 7), (torch.float64, 3)])
def test_message_by_message_and_native_agree_for_every_element_type(fake_ucx, dtype, code):
    """Sixteen-bit floats are folded through float32 and rounded once per addition on both paths:
    three members, values that do not sum exactly, identical bits."""
    torch.manual_seed(11)
    if dtype.is_floating_point:
        values = [(torch.randn(20_011) * 3 ** i).to(dtype) for i in range(3)]
    else:
        values = [torch.randint(-1000, 1000, (20_011,), dtype=dtype) * (i + 1) for i in range(3)]

    def body(worker, i):
        deadline = time.monotonic() + 30
        native, stepwise = values[i].clone(), values[i].clone()
        worker.all_reduce(native.data_ptr(), native.numel(), code, 0, 3_000, 1, deadline)
        tagged.OnDevice(worker, 3, i).all_reduce(stepwise, "sum", 3_000, 2, deadline)
        empty = torch.zeros(0, dtype=dtype)
        tagged.OnDevice(worker, 3, i).all_reduce(empty, "sum", 3_000, 3, deadline)      # nothing to do, nothing posted
        return native.view(torch.uint8).clone(), stepwise.view(torch.uint8).clone()

    out = _workers(3, body)
    for native, stepwise in out:
        assert torch.equal(native, stepwise) and torch.equal(native, out[0][0])


def test_a_ucx_built_for_cuda_memory_opens_the_direct_path_only_where_the_device_allows_it(fake_ucx, monkeypatch):
    from types import SimpleNamespace

    from gpubridge_b200 import gdr
    from gpubridge_b200.rdma_transport import Router
    from gpubridge_b200.ucx.transport import UcxTransport
    monkeypatch.setenv("FAKE_UCP_MEMORY_TYPES", "host,cuda")
    device_tensor = SimpleNamespace(device=SimpleNamespace(type="cuda", index=0), nbytes=1 << 20,
                                    is_contiguous=lambda: True, data_ptr=lambda: 0x1000)

    def body(worker, i):
        assert worker.memory_types() == {"host", "cuda"}
        bridge = UcxTransport(worker, [0, 1], i, timedelta(seconds=5), 1 << 16)
        assert bridge.router.device_registration
        here = bridge.router.route(device_tensor)                   # this machine: whatever its driver says
        ordered = Router(device_registration=True, direct_min_bytes=0,
                         flush_plans=lambda d: gdr.FlushPlan(d, True, False, "ordered"))
        refused = Router(device_registration=True, direct_min_bytes=0,
                         flush_plans=lambda d: gdr.FlushPlan(d, False, False, "unordered writes, no host flush"))
        bridge.worker = None
        return here.how, ordered.route(device_tensor).how, refused.route(device_tensor)

    for here, allowed, refused in _workers(2, body):
        assert here in ("bounce", "in-place") and allowed == "in-place"
        assert refused.how == "bounce" and refused.why == "unordered writes, no host flush"
