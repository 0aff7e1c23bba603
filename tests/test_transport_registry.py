"""The registry of bridge transports: what is loaded when, whose name is whose, and that a
transport swapped in by a user carries every bridged policy.  (Reference: tests/test_transport.py.)"""
import subprocess
import sys

import pytest
import torch

from _harness import LAYOUTS, expected_sum, per_rank, rank_tensor, run_ranks
from gpubridge_b200 import transport


def test_gloo_is_the_default_and_names_and_classes_resolve():
    assert transport.DEFAULT_TRANSPORT == "gloo"
    assert transport.resolve_transport("gloo") is transport.GlooTransport
    assert transport.resolve_transport(transport.GlooTransport) is transport.GlooTransport
    with pytest.raises(TypeError, match="transport name or BridgeTransport subclass"):
        transport.resolve_transport(42)
    with pytest.raises(TypeError):
        transport.resolve_transport(int)
    with pytest.raises(TypeError):
        transport.BridgeTransport()                                # abstract


def test_importing_the_package_loads_no_opt_in_bridge_and_a_name_loads_its_own():
    program = (
        "import sys, gpubridge_b200\n"
        "from gpubridge_b200 import transport\n"
        "opt_in = ['gpubridge_b200.multitcp', 'gpubridge_b200.rdma', 'gpubridge_b200.rdma_transport',\n"
        "          'gpubridge_b200.ucx', 'gpubridge_b200.ucx.transport']\n"
        "assert not [m for m in opt_in if m in sys.modules], [m for m in opt_in if m in sys.modules]\n"
        "transport.resolve_transport('gloo'); transport.resolve_transport('nvlink')\n"
        "assert not [m for m in opt_in if m in sys.modules]\n"
        "try:\n"
        "    transport.resolve_transport('multitcp')\n"
        "except ValueError:\n"
        "    pass\n"
        "assert 'gpubridge_b200.multitcp' in sys.modules\n"
        "assert 'gpubridge_b200.ucx' not in sys.modules and 'gpubridge_b200.rdma_transport' not in sys.modules\n"
        "print('ok')\n")
    done = subprocess.run([sys.executable, "-c", program], capture_output=True, text=True)
    assert done.returncode == 0 and done.stdout.strip() == "ok", done.stderr[-2000:]


@pytest.mark.parametrize("name", ["multitcp", "ucx", "verbs"])
def test_a_built_in_name_stays_the_built_ins_before_it_loads(name):
    class Squatter(transport.GlooTransport):
        pass
    Squatter.name = name
    if name in transport._TRANSPORTS:                              # loaded already in this process: a clash
        with pytest.raises(ValueError, match="already registered"):
            transport.register_transport(Squatter)
        return
    try:
        transport.register_transport(Squatter)
        # whoever registered first under a built-in's name is what the name resolves to: the
        # built-in is not imported over it
        assert transport.resolve_transport(name) is Squatter
    finally:
        transport._TRANSPORTS.pop(name, None)


def test_unknown_names_list_what_is_known():
    with pytest.raises(ValueError) as caught:
        transport.resolve_transport("carrier-pigeon")
    for known in ("gloo", "nvlink", "multitcp", "ucx", "verbs"):
        assert known in str(caught.value)


def test_register_rejects_non_transports_and_name_clashes():
    with pytest.raises(TypeError, match="BridgeTransport subclass"):
        transport.register_transport(object)
    with pytest.raises(TypeError):
        transport.register_transport(transport.GlooTransport(None))            # an instance, not a class

    class Mine(transport.GlooTransport):
        name = "mine-for-this-test"
    try:
        assert transport.register_transport(Mine) is Mine
        assert transport.register_transport(Mine) is Mine          # again: the same class is fine

        class Other(transport.GlooTransport):
            name = "mine-for-this-test"
        with pytest.raises(ValueError, match="already registered"):
            transport.register_transport(Other)
    finally:
        transport._TRANSPORTS.pop("mine-for-this-test", None)


class Relabelled(transport.GlooTransport):
    """A user's transport: Gloo underneath, its own name, and a count of what it carried."""
    name = "relabelled"
    reduce_ops = frozenset({"sum", "max", "min"})
    calls = 0

    def all_reduce(self, tensor, op="sum"):
        Relabelled.calls += 1
        super().all_reduce(tensor, op)

    def broadcast(self, tensor, src):
        Relabelled.calls += 1
        super().broadcast(tensor, src)


def _over_mine(rank, topology):
    import gpubridge_b200 as gb
    assert type(topology.bridge) in (Relabelled, type(None))
    for op, want in ((gb.ReduceOp.SUM, None), (gb.ReduceOp.MAX, None)):
        t = rank_tensor(rank, 999)
        gb.all_reduce(t, op)
        if op == gb.ReduceOp.SUM:
            assert torch.equal(t, expected_sum(topology.world_size, 999))
        else:
            assert torch.equal(t, torch.stack([rank_tensor(r, 999) for r in range(topology.world_size)]).max(0).values)
    t = rank_tensor(rank, 100)
    gb.broadcast(t, 1)
    assert torch.equal(t, rank_tensor(1, 100))
    return Relabelled.calls, topology.peers[rank].bridge


@pytest.mark.parametrize("layout", ["2+2", "3+1"])
@pytest.mark.parametrize("policy", ["reduce-bridge-broadcast", "pipelined-reduce-bridge-broadcast", "sharded-bridge"])
def test_collectives_run_over_a_swapped_in_transport(tmp_path, layout, policy):
    out = run_ranks(LAYOUTS[layout], per_rank, tmp_path, {}, {"bridge": Relabelled, "policy": policy}, _over_mine,
                    mode="plain", timeout=120)
    assert all(name == "relabelled" for _, name in out)
    leaders = [0, 2] if layout == "2+2" else [0, 3]
    assert all(out[r][0] > 0 for r in leaders)                     # the leaders' bridge steps went through it
