"""Where a rank runs and which island it is in, decided from the environment and the torch build:
vendor detection and its override, CPU-only mode, the device of a GPU rank (with a pretend
``torch.cuda``), the identity of the physical GPU, the split-test and island settings - and, as
CPU ranks, that a relabelled job forms its islands, says so on every rank, and is refused when
the ranks disagree or the job is really mixed.  (Reference: tests/test_detect.py,
test_split_test.py, test_topology.py.)"""
import types
import warnings

import pytest
import torch

from _harness import expected_sum, per_rank, rank_tensor, run_ranks
from gpubridge_b200 import config, detect, split_test, topology
from gpubridge_b200.detect import Probe


@pytest.fixture(autouse=True)
def clean_environment(monkeypatch):
    for name in (config.VENDOR_ENV, config.CPU_ONLY_ENV, config.SPLIT_TEST_ENV, config.ISLANDS_ENV,
                 config.SIM_HOSTNAME_ENV, "LOCAL_RANK"):
        monkeypatch.delenv(name, raising=False)


def build(monkeypatch, cuda=None, hip=None):
    monkeypatch.setattr(torch.version, "cuda", cuda, raising=False)
    monkeypatch.setattr(torch.version, "hip", hip, raising=False)


def gpus(monkeypatch, count, current=0):
    monkeypatch.setattr(torch.cuda, "is_available", lambda: count > 0)
    monkeypatch.setattr(torch.cuda, "device_count", lambda: count)
    monkeypatch.setattr(torch.cuda, "current_device", lambda: current)


# ---- vendor ----------------------------------------------------------------------------------------------
@pytest.mark.parametrize("cuda, hip, expected", [("12.8", None, "nvidia"), (None, "6.2", "amd"), ("12.8", "6.2", "amd")])
def test_the_vendor_follows_the_build(monkeypatch, cuda, hip, expected):
    build(monkeypatch, cuda, hip)
    assert detect.detect_hardware_vendor() == detect.detect_vendor() == expected


@pytest.mark.parametrize("value, expected", [("nvidia", "nvidia"), ("AMD", "amd"), ("  amd ", "amd")])
def test_the_override_wins_over_the_build(monkeypatch, value, expected):
    build(monkeypatch, cuda="12.8")
    monkeypatch.setenv(config.VENDOR_ENV, value)
    assert detect.vendor_override() == detect.detect_vendor() == expected
    assert config.is_simulated()                                   # naming a vendor selects CPU simulation


def test_an_empty_override_counts_as_unset_and_an_unknown_one_is_refused(monkeypatch):
    build(monkeypatch, cuda="12.8")
    monkeypatch.setenv(config.VENDOR_ENV, "   ")
    assert detect.vendor_override() is None and detect.detect_vendor() == "nvidia" and not config.is_simulated()
    monkeypatch.setenv(config.VENDOR_ENV, "intel")
    with pytest.raises(ValueError, match="GPUBRIDGE_VENDOR='intel' is not a known vendor.*nvidia"):
        detect.detect_vendor()


def test_a_cpu_build_points_at_simulation_mode(monkeypatch):
    build(monkeypatch)
    with pytest.raises(RuntimeError, match="neither CUDA nor ROCm.*GPUBRIDGE_VENDOR=nvidia"):
        detect.detect_vendor()
    monkeypatch.setenv(config.CPU_ONLY_ENV, "1")                   # CPU-only keeps the BUILD's vendor: none here
    with pytest.raises(RuntimeError, match="GPUBRIDGE_CPU_ONLY does not change that"):
        detect.detect_vendor()
    monkeypatch.setenv(config.VENDOR_ENV, "amd")                   # the override still wins
    assert detect.detect_vendor() == "amd"


@pytest.mark.parametrize("value, expected", [("1", True), ("true", True), ("YES", True), ("on", True),
                                             ("0", False), ("false", False), ("no", False), ("", False)])
def test_cpu_only_flag_values(monkeypatch, value, expected):
    monkeypatch.setenv(config.CPU_ONLY_ENV, value)
    assert config.is_cpu_only() is expected and config.is_simulated() is expected


def test_cpu_only_rejects_what_is_not_a_boolean(monkeypatch):
    monkeypatch.setenv(config.CPU_ONLY_ENV, "maybe")
    with pytest.raises(ValueError, match="GPUBRIDGE_CPU_ONLY='maybe' is not a boolean"):
        config.is_cpu_only()


def test_cpu_only_runs_on_gloo_with_the_builds_vendor(monkeypatch):
    build(monkeypatch, cuda="12.8")
    monkeypatch.setenv(config.CPU_ONLY_ENV, "1")
    cfg = config.resolve_config()
    assert cfg.simulated and cfg.island_backend == "gloo" and cfg.device == torch.device("cpu")
    assert detect.detect_vendor() == "nvidia"


# ---- the device of a GPU rank ---------------------------------------------------------------------------
def test_a_gpu_rank_uses_nccl_on_its_local_rank(monkeypatch):
    gpus(monkeypatch, 8, current=5)
    monkeypatch.setenv("LOCAL_RANK", "3")
    cfg = config.resolve_config()
    assert not cfg.simulated and cfg.island_backend == "nccl" and cfg.device == torch.device("cuda", 3)
    monkeypatch.delenv("LOCAL_RANK")
    assert config.resolve_config().device == torch.device("cuda", 5)          # without it: the current device


@pytest.mark.parametrize("local_rank, count, match", [
    ("8", 8, "LOCAL_RANK=8 asks for GPU 8, but this process sees only 8"),
    ("2", 1, "sees only 1 GPU"), ("-1", 4, "asks for GPU -1"), ("two", 4, "LOCAL_RANK='two' is not an integer")])
def test_a_local_rank_without_a_gpu_is_a_clear_error(monkeypatch, local_rank, count, match):
    gpus(monkeypatch, count)
    monkeypatch.setenv("LOCAL_RANK", local_rank)
    with pytest.raises(RuntimeError, match=match):
        config.resolve_config()


def test_only_a_relabelled_job_may_wrap_around_the_visible_gpus(monkeypatch):
    gpus(monkeypatch, 2)
    monkeypatch.setenv("LOCAL_RANK", "3")
    with pytest.raises(RuntimeError, match="sees only 2"):
        config.resolve_config()
    monkeypatch.setenv(config.SPLIT_TEST_ENV, "half")
    assert config.resolve_config().device == torch.device("cuda", 1)
    monkeypatch.delenv(config.SPLIT_TEST_ENV)
    monkeypatch.setenv(config.ISLANDS_ENV, "2,2")
    assert config.resolve_config().device == torch.device("cuda", 1)


def test_without_a_gpu_the_error_points_at_simulation_mode(monkeypatch):
    gpus(monkeypatch, 0)
    with pytest.raises(RuntimeError, match="No GPU is visible.*GPUBRIDGE_VENDOR=nvidia.*GPUBRIDGE_CPU_ONLY=1"):
        config.resolve_config()


@pytest.mark.parametrize("props, want", [
    (dict(uuid="GPU-1234-abcd", pci_domain_id=0, pci_bus_id=0x1b, pci_device_id=0), "uuid GPU-1234-abcd, pci 0000:1b:00"),
    (dict(uuid="00000000-0000-0000-0000-000000000000", pci_domain_id=1, pci_bus_id=2, pci_device_id=3), "pci 0001:02:03"),
    (dict(uuid="GPU-9"), "uuid GPU-9"), (dict(), ""),
    (dict(uuid="", pci_domain_id=0, pci_bus_id=0, pci_device_id=0), "")])
def test_gpu_identity_is_the_physical_gpu(monkeypatch, props, want):
    monkeypatch.setattr(torch.cuda, "get_device_properties", lambda device: types.SimpleNamespace(**props))
    assert config.gpu_identity(torch.device("cuda", 0)) == want
    assert config.gpu_identity(torch.device("cpu")) is None


def test_gpu_identity_is_empty_when_the_driver_cannot_say(monkeypatch):
    def broken(device):
        raise RuntimeError("driver gone")
    monkeypatch.setattr(torch.cuda, "get_device_properties", broken)
    assert config.gpu_identity(torch.device("cuda", 0)) == ""


def test_a_simulated_hostname_is_ignored_on_gpus(monkeypatch):
    import socket
    monkeypatch.setenv(config.SIM_HOSTNAME_ENV, "pretend")
    assert config.hostname(True) == "pretend" and config.hostname(False) == socket.gethostname()


# ---- split-test and island settings -----------------------------------------------------------------------
@pytest.mark.parametrize("value, mode", [("", None), ("0", None), ("off", None), ("1", "half"), ("true", "half"),
                                         ("half", "half"), ("Alternate", "alternate"), ("node", "node")])
def test_the_variable_is_the_only_switch(monkeypatch, value, mode):
    monkeypatch.setenv(config.SPLIT_TEST_ENV, value)
    assert config.split_test_mode() == mode


def test_an_unknown_split_mode_is_rejected(monkeypatch):
    monkeypatch.setenv(config.SPLIT_TEST_ENV, "thirds")
    with pytest.raises(ValueError, match="GPUBRIDGE_SPLIT_TEST='thirds' is not valid.*half"):
        config.split_test_mode()


@pytest.mark.parametrize("raw, sizes", [("4,4", (4, 4)), ("4+4", (4, 4)), ("2,2,2,2", (2, 2, 2, 2)), ("8", (8,)),
                                        (" 3 , 5 ", (3, 5)), ("", ())])
def test_island_sizes_parse(monkeypatch, raw, sizes):
    monkeypatch.setenv(config.ISLANDS_ENV, raw)
    assert config.islands_setting() == sizes


@pytest.mark.parametrize("raw", ["4,x", "4,,4", "0,8", "-2,10", "4;4"])
def test_bad_island_sizes_are_refused(monkeypatch, raw):
    monkeypatch.setenv(config.ISLANDS_ENV, raw)
    with pytest.raises(ValueError, match="GPUBRIDGE_ISLANDS"):
        config.islands_setting()


@pytest.mark.parametrize("world, mode, flipped", [
    (2, "half", [1]), (3, "half", [2]), (4, "half", [2, 3]), (7, "half", [4, 5, 6]),
    (2, "alternate", [1]), (5, "alternate", [1, 3]), (8, "alternate", [1, 3, 5, 7])])
def test_labels_by_rank(world, mode, flipped):
    labels = split_test.split_labels(["nvidia"] * world, ["h"] * world, mode)
    assert [r for r, label in enumerate(labels) if label == "amd"] == flipped
    other_way = split_test.split_labels(["amd"] * world, ["h"] * world, mode)       # an AMD job flips to nvidia
    assert [r for r, label in enumerate(other_way) if label == "nvidia"] == flipped
    assert len(set(labels)) == 2                                   # always two islands


def test_labels_by_node_follow_machines_in_order_of_first_rank():
    hosts = ["b", "b", "a", "a", "c", "b"]
    labels = split_test.split_labels(["nvidia"] * 6, hosts, "node")
    assert labels == ["nvidia", "nvidia", "amd", "amd", "nvidia", "nvidia"]          # b, a, c -> 0, 1, 0


def test_explicit_islands_take_consecutive_ranks():
    assert split_test.island_labels(["amd"] * 8, (3, 5)) == ["amd"] * 3 + ["nvidia"] * 5
    assert split_test.island_labels(["nvidia"] * 4, (4,)) == ["nvidia"] * 4
    three = split_test.island_labels(["nvidia"] * 6, (1, 2, 3))
    assert three == ["nvidia", "amd", "amd", "nvidia#2", "nvidia#2", "nvidia#2"]
    with pytest.raises(RuntimeError, match="only relabels a single-vendor job"):
        split_test.island_labels(["nvidia", "amd"], (1, 1))


def test_the_banner_names_the_moved_ranks_and_says_what_this_is_not():
    labels = split_test.split_labels(["nvidia"] * 4, ["h"] * 4, "alternate")
    text = split_test.banner("alternate", ["nvidia"] * 4, labels)
    assert "GPUBRIDGE_SPLIT_TEST=alternate" in text and "Ranks [1, 3]" in text and "NOT a mixed-vendor run" in text


# ---- layouts ------------------------------------------------------------------------------------------------
def test_islands_are_ordered_by_leader_and_leaders_are_lowest_ranks():
    layout = topology.plan_topology(["amd", "nvidia", "nvidia", "amd", "nvidia"])
    assert [(i.vendor, i.ranks, i.leader) for i in layout.islands] == [("amd", (0, 3), 0), ("nvidia", (1, 2, 4), 1)]
    assert layout.bridge_ranks == (0, 1)
    again = topology.plan_topology(["amd", "nvidia", "nvidia", "amd", "nvidia"])
    assert again == layout                                         # every rank computes the same thing
    flipped = topology.plan_topology(["nvidia", "amd", "amd", "nvidia", "amd"])
    assert [i.ranks for i in flipped.islands] == [i.ranks for i in layout.islands]
    many = topology.plan_topology(["nvidia", "amd", "nvidia#2", "nvidia#3", "amd"])
    assert len(many.islands) == 4 and many.bridge_ranks == (0, 1, 2, 3)


def _peer(release, build="cu128"):
    probe = Probe("nvidia", f"{release}+{build}", "12.8", None, 1, True, True)
    return topology.PeerInfo(vendor="nvidia", simulated=False, hostname="h", bridge="gloo", probe=probe)


def test_releases_in_the_warning_are_in_version_order():
    with pytest.warns(UserWarning, match=r"2\.9\.1, 2\.10\.0, 2\.11\.0"):
        topology.validate_peers([_peer("2.10.0"), _peer("2.9.1"), _peer("2.11.0")])


def test_the_same_release_on_different_builds_is_quiet():
    with warnings.catch_warnings():
        warnings.simplefilter("error")
        topology.validate_peers([_peer("2.11.0", "cu128"), _peer("2.11.0", "rocm6.2")])
        topology.validate_peers([_peer("2.11.0"), _peer("2.9.0")], warn=False)


# ---- relabelled jobs as CPU ranks -------------------------------------------------------------------------
def _relabelled(rank, topology_):
    import gpubridge_b200 as gb
    t = rank_tensor(rank, 1000)
    gb.all_reduce(t)
    assert torch.equal(t, expected_sum(topology_.world_size, 1000))
    return (topology_.split_test, topology_.run_kind, [i.ranks for i in topology_.layout.islands],
            topology_.vendor, topology_.detected_vendor)


def _warned(rank, world, path, envs, init):
    with warnings.catch_warnings(record=True) as seen:
        warnings.simplefilter("always")
        import gpubridge_b200 as gb
        import os
        from datetime import timedelta
        os.environ.update(envs.get(rank, {}))
        topology_ = gb.init(f"file://{path}", rank=rank, world_size=world, timeout=timedelta(seconds=40), **init)
        try:
            out = _relabelled(rank, topology_)
        finally:
            gb.destroy()
    return out, [str(w.message) for w in seen if issubclass(w.category, gb.SplitTestWarning)]


@pytest.mark.parametrize("mode, islands", [("half", [(0, 1), (2, 3)]), ("alternate", [(0, 2), (1, 3)])])
def test_a_split_run_forms_two_islands_and_every_rank_warns(tmp_path, mode, islands):
    envs = {r: {config.SPLIT_TEST_ENV: mode} for r in range(4)}
    out = run_ranks(("nvidia",) * 4, _warned, tmp_path, envs, {}, mode="plain", timeout=90)
    for rank, ((split, kind, got, label, detected), warned) in enumerate(out):
        assert split == mode and got == islands and "split" in kind
        assert detected == "nvidia" and label == ("amd" if rank in islands[1] else "nvidia")
        assert len(warned) == 1 and "NOT a mixed-vendor run" in warned[0]


def test_node_mode_splits_by_simulated_machine(tmp_path):
    envs = {r: {config.SPLIT_TEST_ENV: "node", config.SIM_HOSTNAME_ENV: f"box{r // 2}"} for r in range(4)}
    out = run_ranks(("amd",) * 4, per_rank, tmp_path, envs, {}, _relabelled, mode="plain", timeout=90)
    assert all(o[2] == [(0, 1), (2, 3)] for o in out) and [o[3] for o in out] == ["amd", "amd", "nvidia", "nvidia"]


def test_a_normal_run_is_not_marked_as_split(tmp_path):
    out = run_ranks(("nvidia", "nvidia", "amd"), _warned, tmp_path, {}, {}, mode="plain", timeout=90)
    assert all(o[0][0] is None and "split" not in o[0][1] and o[1] == [] for o in out)


@pytest.mark.parametrize("what, vendors, envs, message", [
    ("ranks disagree on the mode", ("nvidia",) * 4, {0: {"GPUBRIDGE_SPLIT_TEST": "half"}}, "disagree on GPUBRIDGE_SPLIT_TEST"),
    ("a really mixed job", ("nvidia", "nvidia", "amd", "amd"), {r: {"GPUBRIDGE_SPLIT_TEST": "half"} for r in range(4)},
     "only splits a single-vendor job"),
    ("node mode on one machine", ("nvidia",) * 4, {r: {"GPUBRIDGE_SPLIT_TEST": "node"} for r in range(4)},
     "every rank runs on"),
    ("an unknown mode on one rank", ("nvidia",) * 4, {2: {"GPUBRIDGE_SPLIT_TEST": "thirds"}}, "is not valid"),
    ("island sizes that do not add up", ("nvidia",) * 4, {r: {"GPUBRIDGE_ISLANDS": "3,3"} for r in range(4)},
     "names 6 ranks but the job has 4"),
])
def test_splits_that_cannot_be_are_refused_on_every_rank(tmp_path, what, vendors, envs, message):
    errors = run_ranks(vendors, per_rank, tmp_path, envs, {}, mode="plain", expect_error=message, timeout=90)
    assert len(errors) == len(vendors)
