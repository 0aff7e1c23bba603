"""The ``verbs`` bridge over the in-process fabric: routing of tensors (in place / plain /
bounce), the registered staging pool, piecewise bouncing, and the flush decision for direct
receives into device memory (with a fake driver)."""
import threading
from datetime import timedelta

import pytest
import torch

from gpubridge_b200 import gdr, rdma
from gpubridge_b200.rdma_transport import RdmaTransport, RegisteredStaging, Router

from gpubridge_b200.ops import _lib

pytestmark = pytest.mark.skipif(not _lib.available(), reason="the native library is not built")


def _members(count, body, **settings):
    """Run ``body(transport, index)`` on ``count`` members of one fabric, one thread each."""
    fabric = rdma.MockFabric(count)
    members = list(range(10, 10 + count))
    bridges = [RdmaTransport.over_fabric(fabric, members, m, timeout=timedelta(seconds=20), **settings)
               for m in members]
    out, errors = [None] * count, []

    def run(i):
        try:
            out[i] = body(bridges[i], i)
        except BaseException as failure:  # noqa: BLE001
            errors.append((i, failure))

    threads = [threading.Thread(target=run, args=(i,)) for i in range(count)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(60)
    described = [b.describe() for b in bridges]
    for b in bridges:
        b.close()
    fabric.close()
    assert not errors, errors
    return out, described


# ---- the router --------------------------------------------------------------------------------
class _Plans:
    def __init__(self, direct_ok, reason="fake"):
        self.direct_ok, self.reason = direct_ok, reason

    def __call__(self, device):
        return gdr.FlushPlan(device, self.direct_ok, False, self.reason)


class _DeviceTensor:
    """What the router looks at, for a tensor on a device this box does not have."""

    def __init__(self, nbytes, contiguous=True):
        self.nbytes, self._c = nbytes, contiguous
        self.device = torch.device("cuda", 1)

    def is_contiguous(self):
        return self._c


def test_router_host_tensors_go_as_they_lie_and_strided_ones_bounce():
    router = Router()
    assert router.route(torch.zeros(10)).how == "plain"
    assert router.route(torch.zeros(4, 4).t()).how == "bounce"
    assert router.counts == {"plain": 1, "bounce": 1}


def test_router_device_tensors():
    no_registration = Router(device_registration=False)
    assert no_registration.route(_DeviceTensor(1 << 20)).how == "bounce"
    direct = Router(device_registration=True, direct_min_bytes=4096, flush_plans=_Plans(True))
    assert direct.route(_DeviceTensor(1 << 20)).how == "in-place"
    small = direct.route(_DeviceTensor(100))
    assert small.how == "bounce" and "cheaper" in small.why
    refused = Router(device_registration=True, direct_min_bytes=0, flush_plans=_Plans(False, "no flush"))
    route = refused.route(_DeviceTensor(1 << 20))
    assert route.how == "bounce" and route.why == "no flush"


# ---- the flush decision ---------------------------------------------------------------------------
class _FakeDriver:
    def __init__(self, supported=1, ordering=0, options=1, fail=False):
        self.values = {"GPU_DIRECT_RDMA_SUPPORTED": supported,
                       "GPU_DIRECT_RDMA_WRITES_ORDERING": ordering,
                       "GPU_DIRECT_RDMA_FLUSH_WRITES_OPTIONS": options}
        self.fail, self.flushes = fail, 0

    def attribute(self, device, name):
        if self.fail:
            raise RuntimeError("unknown attribute")
        return self.values[name]

    def flush_owner(self):
        self.flushes += 1


@pytest.mark.parametrize("driver, direct, flush", [
    (_FakeDriver(supported=0), False, False),
    (_FakeDriver(ordering=gdr.ORDER_OWNER), True, False),
    (_FakeDriver(ordering=gdr.ORDER_ALL), True, False),
    (_FakeDriver(ordering=gdr.ORDER_NONE, options=1), True, True),
    (_FakeDriver(ordering=gdr.ORDER_NONE, options=0), False, False),
    (_FakeDriver(fail=True), False, False),
])
def test_flush_plan(driver, direct, flush):
    plan = gdr.plan(0, driver)
    assert (plan.direct_ok, plan.flush_needed) == (direct, flush), plan.reason
    plan.after_receive()
    assert driver.flushes == (1 if flush else 0)
    assert plan.describe()["reason"]


def test_plan_without_a_driver_refuses_direct_receives():
    plan = gdr.plan(7)
    if not torch.cuda.is_available():
        assert not plan.direct_ok and not plan.flush_needed


# ---- staging ----------------------------------------------------------------------------------------
class _CountingEndpoint:
    def __init__(self):
        self.dropped = []

    def invalidate(self, ptr, nbytes):
        self.dropped.append((ptr, nbytes))
        return 1


def test_staging_reuses_size_classes_and_evicts_the_oldest():
    endpoint = _CountingEndpoint()
    pool = RegisteredStaging(endpoint, budget_bytes=3 << 20, pin=False)
    a = pool.take(1 << 20)
    assert pool.take((1 << 20) - 5).data_ptr() == a.data_ptr() and pool.reused == 1
    b = pool.take(2 << 20)
    assert pool.held_bytes() == 3 << 20 and not endpoint.dropped
    pool.take(1 << 20)                       # touch a: b is now the oldest
    c = pool.take(1 << 19)                   # over budget: b goes
    assert endpoint.dropped == [(b.data_ptr(), 2 << 20)] and pool.evicted == 1
    assert pool.held_bytes() == (1 << 20) + (1 << 19) and c.numel() == 1 << 19
    pool.close()
    assert len(endpoint.dropped) == 3 and pool.held_bytes() == 0


# ---- the bridge --------------------------------------------------------------------------------------
@pytest.mark.parametrize("count", [2, 3])
def test_host_tensors_are_reduced_in_place(count):
    def body(bridge, i):
        t = torch.arange(50_000, dtype=torch.float32) + i
        bridge.all_reduce(t)
        b = torch.full((1000,), float(i))
        bridge.broadcast(b, bridge.members[1])
        return t, b

    out, described = _members(count, body)
    want = count * torch.arange(50_000, dtype=torch.float32) + sum(range(count))
    for t, b in out:
        assert torch.equal(t, want) and torch.equal(b, torch.full((1000,), 1.0))
    assert all(d["routes"] == {"plain": 2} for d in described)


def test_strided_tensors_bounce_in_pieces_and_come_back():
    def body(bridge, i):
        base = torch.zeros(300, 70)
        t = base.t()                                    # not contiguous
        t += torch.arange(300, dtype=torch.float32) + i
        bridge.all_reduce(t)
        b = torch.zeros(64, 33).t()
        if i == 0:
            b += 5.0
        bridge.broadcast(b, bridge.members[0])
        return t.clone(), b.clone()

    out, described = _members(2, body, piece_bytes=16 << 10)
    want = (2 * torch.arange(300, dtype=torch.float32) + 1).expand(70, 300)
    for t, b in out:
        assert torch.equal(t, want)
        assert torch.equal(b, torch.full((33, 64), 5.0))
    for d in described:
        assert d["routes"] == {"bounce": 2}
        assert d["staging"]["allocated"] >= 1 and d["staging"]["reused"] >= 1
        sent = d["endpoint"]["eager_sent"] + d["endpoint"]["rndv_sent"]
        assert sent > 2                                     # several pieces, each its own call


def test_a_failure_breaks_the_bridge_for_both_members():
    fabric = rdma.MockFabric(2)
    bridges = [RdmaTransport.over_fabric(fabric, [0, 1], m, timeout=timedelta(seconds=3)) for m in (0, 1)]
    fabric.inject("error", src=0, dst=1, nth=1)
    errors = []

    def run(i):
        try:
            bridges[i].all_reduce(torch.ones(1 << 16))
        except RuntimeError as failure:
            errors.append(str(failure))

    threads = [threading.Thread(target=run, args=(i,)) for i in (0, 1)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(30)
    assert len(errors) == 2
    with pytest.raises(RuntimeError):
        bridges[0].all_reduce(torch.ones(8))            # broken stays broken
    for b in bridges:
        b.close()
    fabric.close()


def test_the_name_still_says_why_it_cannot_load():
    from gpubridge_b200 import transport
    with pytest.raises(ValueError, match="provider"):
        transport.resolve_transport("verbs")


def test_the_command_lines_say_what_this_build_has():
    import json
    import subprocess
    import sys
    done = subprocess.run([sys.executable, "-m", "gpubridge_b200.rdma", "info"], capture_output=True, text=True)
    told = json.loads(done.stdout)
    assert told["protocol"] >= 1 and told["in_process_fabric"] and told["provider"] is None
