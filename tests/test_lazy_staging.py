"""The pipelined bridge's copy ordering, checked on CPU with deferred copies: results equal
flat-gloo only if every copy the bridge depends on was waited for; slots are reused across
collectives only after their last copy back; a staging layer that skips the host wait is
caught (the negative control)."""
import pytest
import torch

from _harness import LAYOUTS, expected_sum, rank_tensor, run_ranks


def _install(topology, cls):
    from gpubridge_b200.policies import PipelinedReduceBridgeBroadcast
    policy = topology.policy
    assert isinstance(policy, PipelinedReduceBridgeBroadcast)
    if topology.is_leader and topology.layout.needs_bridge:
        policy.staging = cls(policy.chunk_bytes, policy.SLOTS)
        policy.copied_back = [None] * policy.SLOTS
    return policy


def _deferred(rank, topology, kind):
    import gpubridge_b200 as gb
    import _staging
    cls = getattr(_staging, kind)
    policy = _install(topology, cls)
    world = topology.world_size
    if isinstance(policy.staging, _staging.CallerKeepsGoing):
        # an island collective is queued on the caller's stream, i.e. behind the waits that
        # end() left there: on CPU, let that stream catch up before the island group reads
        island, staging = topology.island_group, policy.staging
        for name in ("broadcast", "all_reduce", "reduce"):
            original = getattr(island, name)

            def ordered(*a, _original=original, **k):
                staging.caller_reaches_the_waits()
                return _original(*a, **k)
            setattr(island, name, ordered)
    failures = []
    for n in (1, 1000, 5000, 20_000):          # 1, 1, 2 and 5 chunks of 4096 floats
        t = rank_tensor(rank, n)
        gb.all_reduce(t)
        if isinstance(policy.staging, _staging.CallerKeepsGoing):
            policy.staging.caller_reaches_the_waits()
        if not torch.equal(t, expected_sum(world, n)):
            failures.append(n)
        t = rank_tensor(rank, n)
        gb.broadcast(t, world - 1)
        if isinstance(policy.staging, _staging.CallerKeepsGoing):
            policy.staging.caller_reaches_the_waits()
        if not torch.equal(t, rank_tensor(world - 1, n)):
            failures.append(-n)
    journal = list(policy.staging.journal) if isinstance(policy.staging, _staging.DeferredStaging) else []
    return failures, journal


@pytest.mark.parametrize("kind", ["DeferredStaging", "CallerKeepsGoing"])
def test_every_needed_copy_is_waited_for(tmp_path, kind):
    out = run_ranks(LAYOUTS["2+2"], _deferred, tmp_path, kind,
                    init={"policy": "pipelined-reduce-bridge-broadcast"},
                    env={"GPUBRIDGE_CHUNK_BYTES": "16K"})
    for rank, (failures, journal) in enumerate(out):
        assert failures == [], (rank, failures)
    leader_journal = out[0][1]
    ran = [e[1] for e in leader_journal if e[0] == "ran"]
    queued = [e[1] for e in leader_journal if e[0] == "to_host"] + \
             [e[1] for e in leader_journal if e[0] == "to_device"]
    assert ran and set(ran) <= set(queued)
    # a slot's next copy out names the last copy back out of the same slot as its precondition
    gated = [e for e in leader_journal if e[0] == "to_host" and e[2] is not None]
    assert gated and all(e[2].startswith("back") for e in gated)


def test_a_skipped_host_wait_is_caught(tmp_path):
    out = run_ranks(LAYOUTS["2+2"], _deferred, tmp_path, "SkipsWaitHost",
                    init={"policy": "pipelined-reduce-bridge-broadcast"},
                    env={"GPUBRIDGE_CHUNK_BYTES": "16K"})
    assert any(failures for failures, _ in out), "the bridge read slots whose copies never ran"
