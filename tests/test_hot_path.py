"""What the per-call path caches, and that caching never changes an answer: the policy's list of
reduce operations is asked once per (policy, topology) yet every call is still checked against
it; a new topology never inherits an old topology's answer; reduce operations are named by a
dictionary hit for the enum members and by comparison for the instances torch builds at run
time; validation runs on every call.  (The reference pins the same properties:
tests/test_hot_path.py.)"""
import gc
import types

import pytest
import torch
from torch.distributed import ReduceOp

from gpubridge_b200 import collectives as C


class CountingPolicy:
    name = "counting"

    def __init__(self, ops=("sum", "max")):
        self.asked, self.ops = 0, frozenset(ops)

    def supported_reduce_ops(self, topology):
        self.asked += 1
        return self.ops


class SlottedPolicy:
    """A policy that cannot carry the cache attribute: it is simply asked every time."""
    __slots__ = ("asked",)
    name = "slotted"

    def __init__(self):
        self.asked = 0

    def supported_reduce_ops(self, topology):
        self.asked += 1
        return frozenset({"sum"})


class _Topology:
    """As much of a Topology as validation reads (a class of its own: it can be weakly referenced)."""

    def __init__(self):
        self.rank, self.peers = 0, [types.SimpleNamespace(bridge="gloo")]
        self.device, self.simulated, self.world_size = torch.device("cpu"), True, 2


def _topology():
    return _Topology()


def test_the_policy_is_asked_once_and_every_call_is_still_checked():
    policy, topology = CountingPolicy(), _topology()
    for _ in range(50):
        C._check_reduce_op(policy, "sum", topology, "all_reduce")
        C._check_reduce_op(policy, "max", topology, "all_reduce")
    assert policy.asked == 1
    for _ in range(3):                                   # an unsupported op is refused every time
        with pytest.raises(NotImplementedError, match="MIN.*supports only MAX, SUM"):
            C._check_reduce_op(policy, "min", topology, "all_reduce")
    assert policy.asked == 1


def test_a_new_topology_is_never_given_an_old_answer():
    policy = CountingPolicy()
    first = _topology()
    C._check_reduce_op(policy, "sum", first, "all_reduce")
    policy.ops = frozenset({"max"})                      # what the next topology supports
    second = _topology()
    with pytest.raises(NotImplementedError):
        C._check_reduce_op(policy, "sum", second, "all_reduce")
    assert policy.asked == 2
    # even when the old topology's memory is reused for a new object
    del first, second
    gc.collect()
    third = _topology()
    policy.ops = frozenset({"sum"})
    C._check_reduce_op(policy, "sum", third, "all_reduce")
    assert policy.asked == 3


def test_a_policy_that_cannot_hold_the_cache_is_asked_every_call():
    policy, topology = SlottedPolicy(), _topology()
    for _ in range(5):
        C._check_reduce_op(policy, "sum", topology, "all_reduce")
    assert policy.asked == 5


def test_reduce_ops_are_named_by_lookup_and_by_comparison():
    for op, name in ((ReduceOp.SUM, "sum"), (ReduceOp.AVG, "avg"), (ReduceOp.MAX, "max"), (ReduceOp.MIN, "min")):
        assert C._op_name(op, "all_reduce") == name
        assert C._op_name(ReduceOp(op), "all_reduce") == name       # the instance torch passes backends
    for bad in (ReduceOp.PRODUCT, ReduceOp.BAND, ReduceOp.BXOR, "product", None):
        with pytest.raises(ValueError, match="supports ReduceOp.SUM, AVG, MAX and MIN"):
            C._op_name(bad, "all_reduce")


def test_tensors_are_validated_on_every_call():
    topology = _topology()
    good = torch.ones(4)
    for _ in range(3):
        C._check_tensor(good, topology)
    with pytest.raises(TypeError):
        C._check_tensor([1.0], topology)
    with pytest.raises(ValueError, match="doesn't support torch.complex64"):
        C._check_tensor(torch.ones(2, dtype=torch.complex64), topology)
    with pytest.raises(ValueError, match="contiguous"):
        C._check_tensor(torch.ones(4, 4)[:, 1], topology)
    with pytest.raises(ValueError, match="AVG needs a floating-point"):
        C._check_avg("avg", torch.int32, "all_reduce")
    C._check_avg("avg", torch.bfloat16, "all_reduce")
    C._check_avg("sum", torch.int32, "all_reduce")


def test_sizes_of_gather_and_scatter_are_checked_against_the_world():
    topology = _topology()
    C._check_pair(torch.empty(8), torch.empty(4), topology, "all_gather_into_tensor",
                  big=torch.empty(8), small=torch.empty(4))
    with pytest.raises(ValueError, match="world_size"):
        C._check_pair(torch.empty(9), torch.empty(4), topology, "all_gather_into_tensor",
                      big=torch.empty(9), small=torch.empty(4))
    with pytest.raises(ValueError, match="output is torch.float64 but input is torch.float32"):
        C._check_pair(torch.empty(8, dtype=torch.float64), torch.empty(4), topology, "x",
                      big=torch.empty(8), small=torch.empty(4))
