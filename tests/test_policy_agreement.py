"""What the ranks of a job must agree on before a policy runs, and what each bridged policy puts
on its links: different policies, chunk sizes or thresholds files on different ranks fail init on
EVERY rank with the same explanation; a thresholds file steers the auto-tuned policy by size;
the sharded bridge gives every link one stripe; the pipelined bridge cuts the bridge step into
its chunks.  Ranks are CPU processes; the links are watched by a transport that counts.
(Reference: tests/test_policies.py, test_pipelined.py, test_sharded.py.)"""
import json

import pytest
import torch

from _harness import LAYOUTS, expected_sum, per_rank, rank_tensor, run_ranks
from gpubridge_b200 import policies, transport


class CountingGloo(transport.GlooTransport):
    """Gloo links that write down what they carried (per process: one rank's view)."""
    name = "counting-gloo"
    carried: list = []

    def all_reduce(self, tensor, op="sum"):
        CountingGloo.carried.append(("all_reduce", tuple(self.group.ranks), tensor.numel()))
        super().all_reduce(tensor, op)

    def broadcast(self, tensor, src):
        CountingGloo.carried.append(("broadcast", tuple(self.group.ranks), tensor.numel()))
        super().broadcast(tensor, src)


transport.register_transport(CountingGloo)


# ---- before anything is joined ------------------------------------------------------------------------
def test_init_rejects_an_unknown_policy_or_bridge_before_joining():
    import gpubridge_b200 as gb
    with pytest.raises(ValueError, match="unknown collective policy"):
        gb.init("file:///nonexistent/never-touched", rank=0, world_size=2, policy="fastest")
    with pytest.raises(ValueError, match="unknown bridge transport"):
        gb.init("file:///nonexistent/never-touched", rank=0, world_size=2, bridge="carrier-pigeon")


def test_collective_policy_is_abstract_and_flat_gloo_fits_every_layout():
    from gpubridge_b200 import topology
    with pytest.raises(TypeError):
        policies.CollectivePolicy()
    for vendors in (["nvidia"], ["nvidia", "amd"], ["nvidia", "nvidia", "amd"], ["amd"] * 5):
        layout = topology.plan_topology(vendors)
        assert policies.FlatGloo.applies_to(layout)
        assert policies.AutoTuned.applies_to(layout)
        bridged = len(set(vendors)) > 1
        assert policies.ReduceBridgeBroadcast.applies_to(layout) == bridged
        assert policies.NativeOnly.applies_to(layout) == (not bridged)
        picked = policies.choose_policy("auto", layout)
        assert picked is (policies.ReduceBridgeBroadcast if bridged else policies.NativeOnly)
        assert picked is not policies.ShardedBridge                 # auto never picks the sharded bridge


# ---- disagreement between ranks: every rank learns of it ------------------------------------------------
@pytest.mark.parametrize("what, envs, inits, message", [
    ("policies", {}, {1: {"policy": "flat-gloo"}}, "picked different collective policies"),
    ("chunk sizes", {2: {"GPUBRIDGE_CHUNK_BYTES": "1M"}}, {}, "disagree on the settings of collective policy"),
    ("a bad chunk size", {3: {"GPUBRIDGE_CHUNK_BYTES": "12"}}, {}, "multiple of 8"),
    ("pinned staging", {0: {"GPUBRIDGE_PINNED_STAGING": "1"}}, {}, "GPUBRIDGE_PINNED_STAGING"),
    ("codec formats", {1: {"GPUBRIDGE_CODEC_FORMAT": "b200"}}, {}, "GPUBRIDGE_CODEC_FORMAT"),
    ("bridges", {}, {2: {"bridge": "counting-gloo"}}, "picked different bridge transports"),
])
def test_ranks_that_disagree_fail_init_on_every_rank(tmp_path, what, envs, inits, message):
    errors = run_ranks(LAYOUTS["2+2"], _join, tmp_path, envs, inits, "pipelined-reduce-bridge-broadcast",
                       mode="plain", expect_error=message, timeout=90)
    assert len(errors) == 4


def _join(rank, world, path, envs, inits, policy):
    return per_rank(rank, world, path, envs, dict({"policy": policy}, **inits.get(rank, {})))


@pytest.mark.parametrize("layout, policy", [("single-vendor", "reduce-bridge-broadcast"),
                                            ("single-vendor", "sharded-bridge"), ("2+2", "native-only")])
def test_a_policy_that_does_not_fit_fails_init_on_every_rank(tmp_path, layout, policy):
    run_ranks(LAYOUTS[layout], _join, tmp_path, {}, {}, policy, mode="plain", expect_error="doesn't apply", timeout=90)


# ---- thresholds files -----------------------------------------------------------------------------------
RULES = [{"max_bytes": 4096, "policy": "flat-gloo"},
         {"max_bytes": 1 << 20, "policy": "reduce-bridge-broadcast"},
         {"max_bytes": None, "policy": "sharded-bridge"}]


def _thresholds(tmp_path, rules=RULES, name="t.json", chunk=1 << 20):
    path = tmp_path / name
    policies.write_thresholds(str(path), rules, chunk)
    return str(path)


def _which_policy_by_size(rank, topology):
    import gpubridge_b200 as gb
    picked = {}
    for numel in (8, 1024, 1025, 100_000, 300_000):
        picked[numel * 4] = topology.policy.select_policy(numel * 4).name
        t = rank_tensor(rank, numel)
        gb.all_reduce(t)
        assert torch.equal(t, expected_sum(topology.world_size, numel))
    return picked


def test_auto_tuned_follows_the_thresholds_file(tmp_path):
    path = _thresholds(tmp_path)
    out = run_ranks(LAYOUTS["2+2"], per_rank, tmp_path, {r: {"GPUBRIDGE_THRESHOLDS": path} for r in range(4)},
                    {"policy": "auto-tuned"}, _which_policy_by_size, mode="plain", timeout=120)
    assert out[0] == {32: "flat-gloo", 4096: "flat-gloo", 4100: "reduce-bridge-broadcast",
                      400_000: "reduce-bridge-broadcast", 1_200_000: "sharded-bridge"}
    assert all(o == out[0] for o in out)


def test_auto_tuned_without_a_file_does_what_auto_does(tmp_path):
    out = run_ranks(LAYOUTS["3+1"], per_rank, tmp_path, {}, {"policy": "auto-tuned"}, _which_policy_by_size,
                    mode="plain", timeout=120)
    assert set(out[0].values()) == {"reduce-bridge-broadcast"}


def test_identical_files_at_different_paths_agree(tmp_path):
    envs = {r: {"GPUBRIDGE_THRESHOLDS": _thresholds(tmp_path, name=f"copy-{r}.json")} for r in range(4)}
    assert run_ranks(LAYOUTS["2+2"], per_rank, tmp_path, envs, {"policy": "auto-tuned"}, mode="plain",
                     timeout=90) == ["up"] * 4


@pytest.mark.parametrize("what, change, message", [
    ("different rules", lambda tmp: {1: {"GPUBRIDGE_THRESHOLDS": _thresholds(
        tmp, [{"max_bytes": None, "policy": "flat-gloo"}], "other.json")}}, "disagree on the settings"),
    ("a different chunk size in the file", lambda tmp: {2: {"GPUBRIDGE_THRESHOLDS": _thresholds(
        tmp, RULES, "chunk.json", chunk=1 << 16)}}, "disagree on the settings"),
    ("a file that is missing on one rank", lambda tmp: {3: {"GPUBRIDGE_THRESHOLDS": str(tmp / "nowhere.json")}},
     "can't read it"),
    ("no file on one rank", lambda tmp: {0: {"GPUBRIDGE_THRESHOLDS": ""}}, "disagree on the settings"),
])
def test_ranks_with_different_thresholds_fail_init_on_every_rank(tmp_path, what, change, message):
    path = _thresholds(tmp_path)
    envs = {r: {"GPUBRIDGE_THRESHOLDS": path} for r in range(4)}
    envs.update(change(tmp_path))
    errors = run_ranks(LAYOUTS["2+2"], per_rank, tmp_path, envs, {"policy": "auto-tuned"}, mode="plain",
                       expect_error=message, timeout=90)
    assert len(errors) == 4


def test_a_rule_that_does_not_fit_the_cluster_fails_init_on_every_rank(tmp_path):
    path = _thresholds(tmp_path, [{"max_bytes": None, "policy": "sharded-bridge"}])
    run_ranks(LAYOUTS["single-vendor"], per_rank, tmp_path, {r: {"GPUBRIDGE_THRESHOLDS": path} for r in range(3)},
              {"policy": "auto-tuned"}, mode="plain", expect_error="can't be used here", timeout=90)


def test_a_thresholds_file_is_plain_json_with_a_format_number(tmp_path):
    path = _thresholds(tmp_path)
    with open(path) as fh:
        written = json.load(fh)
    assert written["gpubridge_thresholds"] == policies.THRESHOLDS_FORMAT == 1
    assert written["rules"] == RULES and written["chunk_bytes"] == 1 << 20
    written["gpubridge_thresholds"] = 2
    with open(path, "w") as fh:
        json.dump(written, fh)
    with pytest.raises(ValueError, match="format|version|thresholds file"):
        policies.load_thresholds(path, 1 << 20)


# ---- what the links carry -------------------------------------------------------------------------------
def _carried(rank, topology, numel):
    import gpubridge_b200 as gb
    CountingGloo.carried.clear()
    t = rank_tensor(rank, numel)
    gb.all_reduce(t)
    assert torch.equal(t, expected_sum(topology.world_size, numel))
    return list(CountingGloo.carried)


@pytest.mark.parametrize("layout, k", [("2+2", 2), ("3+1", 1), ("interleaved", 2)])
def test_each_link_of_the_sharded_bridge_carries_one_stripe(tmp_path, layout, k):
    numel = 10_001
    out = run_ranks(LAYOUTS[layout], per_rank, tmp_path, {}, {"policy": "sharded-bridge", "bridge": "counting-gloo"},
                    _carried, numel, mode="plain", timeout=120)
    stripe = -(-numel // k)
    links = set()
    for rank, seen in enumerate(out):
        reduces = [entry for entry in seen if entry[0] == "all_reduce"]
        assert len(reduces) <= 1                                    # a rank is on one link at most
        for _, members, carried in reduces:
            assert carried == stripe and rank in members
            links.add(members)
    assert len(links) == k                                          # k links, each between one rank per island
    vendors = LAYOUTS[layout]
    for members in links:
        assert sorted(vendors[m] for m in members) == ["amd", "nvidia"]


def test_the_reduce_bridge_broadcast_bridge_step_is_one_message_between_the_leaders(tmp_path):
    out = run_ranks(LAYOUTS["2+2"], per_rank, tmp_path, {}, {"policy": "reduce-bridge-broadcast",
                    "bridge": "counting-gloo"}, _carried, 50_000, mode="plain", timeout=120)
    assert out[0] == out[2] == [("all_reduce", (0, 2), 50_000)] and out[1] == out[3] == []


def test_the_pipelined_bridge_step_goes_chunk_by_chunk(tmp_path):
    envs = {r: {"GPUBRIDGE_CHUNK_BYTES": "64K"} for r in range(4)}
    out = run_ranks(LAYOUTS["2+2"], per_rank, tmp_path, envs, {"policy": "pipelined-reduce-bridge-broadcast",
                    "bridge": "counting-gloo"}, _carried, 50_000, mode="plain", timeout=120)
    per_chunk = (64 << 10) // 4
    want = [per_chunk] * (50_000 // per_chunk) + [50_000 % per_chunk]
    assert [n for _, _, n in out[0]] == want and out[0] == out[2] and out[1] == out[3] == []
