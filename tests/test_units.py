"""Pure unit tests: configuration parsing, detection, split labels, layout planning, peer
validation, policy registry and thresholds files (reference: tests/test_detect.py,
test_split_test.py, test_policies.py, test_probe.py)."""
import json

import pytest
import torch

from gpubridge_b200 import config, detect, policies, split_test, topology, transport
from gpubridge_b200.detect import Probe


def test_parse_size_and_settings(monkeypatch):
    assert config.parse_size("4M") == 4 << 20 and config.parse_size("64kb") == 64 << 10
    assert config.parse_size("1G") == 1 << 30 and config.parse_size("65536") == 65536
    with pytest.raises(ValueError):
        config.parse_size("lots")
    monkeypatch.setenv(config.CHUNK_BYTES_ENV, "12")
    with pytest.raises(ValueError, match="multiple of 8"):
        config.chunk_bytes_setting(4 << 20)
    monkeypatch.setenv(config.CHUNK_BYTES_ENV, "1M")
    assert config.chunk_bytes_setting(4 << 20) == 1 << 20
    monkeypatch.setenv(config.PINNED_STAGING_ENV, "maybe")
    with pytest.raises(ValueError, match="not a boolean"):
        config.pinned_staging_setting()
    monkeypatch.setenv(config.BRIDGE_COMPRESSION_ENV, "FP8")
    assert config.bridge_compression_setting() == "fp8"
    monkeypatch.setenv(config.BRIDGE_COMPRESSION_ENV, "off")
    assert config.bridge_compression_setting() == ""
    monkeypatch.setenv(config.BRIDGE_COMPRESSION_ENV, "int4")
    with pytest.raises(ValueError):
        config.bridge_compression_setting()
    monkeypatch.setenv(config.SPLIT_TEST_ENV, "1")
    assert config.split_test_mode() == "half"
    monkeypatch.setenv(config.SPLIT_TEST_ENV, "thirds")
    with pytest.raises(ValueError):
        config.split_test_mode()
    monkeypatch.setenv(config.ISLANDS_ENV, "4+4")
    assert config.islands_setting() == (4, 4)
    monkeypatch.setenv(config.ISLANDS_ENV, "4,x")
    with pytest.raises(ValueError):
        config.islands_setting()


def test_simulation_config(monkeypatch):
    monkeypatch.setenv(config.VENDOR_ENV, "amd")
    monkeypatch.setenv(config.SIM_HOSTNAME_ENV, "node7")
    cfg = config.resolve_config()
    assert cfg.simulated and cfg.island_backend == "gloo" and cfg.device.type == "cpu"
    assert config.hostname(True) == "node7" and config.gpu_identity(cfg.device) is None
    assert detect.detect_vendor() == "amd"
    monkeypatch.setenv(config.VENDOR_ENV, "intel")
    with pytest.raises(ValueError, match="not a known vendor"):
        detect.detect_vendor()


def test_no_gpu_is_a_clear_error(monkeypatch):
    monkeypatch.setattr(torch.cuda, "is_available", lambda: False)
    with pytest.raises(RuntimeError, match="No GPU is visible"):
        config.resolve_config()


def test_probe_never_raises(monkeypatch):
    def boom():
        raise OSError("driver on fire")
    monkeypatch.setattr(torch.cuda, "device_count", boom)
    result = detect.probe()
    assert result.gpu_count == 0 and any("driver on fire" in e for e in result.errors)
    assert result.torch_version == str(torch.__version__)


def test_split_labels():
    v = ["nvidia"] * 5
    h = ["a", "a", "b", "b", "c"]
    assert split_test.split_labels(v, h, "half") == ["nvidia"] * 3 + ["amd"] * 2
    assert split_test.split_labels(v, h, "alternate") == ["nvidia", "amd"] * 2 + ["nvidia"]
    assert split_test.split_labels(v, h, "node") == ["nvidia", "nvidia", "amd", "amd", "nvidia"]
    with pytest.raises(RuntimeError, match="at least 2"):
        split_test.split_labels(["amd"], ["a"], "half")
    with pytest.raises(RuntimeError, match="single-vendor"):
        split_test.split_labels(["amd", "nvidia"], ["a", "a"], "half")
    with pytest.raises(RuntimeError, match="every rank runs on"):
        split_test.split_labels(["amd", "amd"], ["a", "a"], "node")
    labels = split_test.island_labels(["nvidia"] * 8, (2, 2, 2, 2))
    assert labels == ["nvidia"] * 2 + ["amd"] * 2 + ["nvidia#2"] * 2 + ["nvidia#3"] * 2
    with pytest.raises(RuntimeError, match="names 6 ranks"):
        split_test.island_labels(["nvidia"] * 8, (3, 3))
    assert "NOT a mixed-vendor run" in split_test.banner("half", v, split_test.split_labels(v, h, "half"))


def test_plan_topology():
    layout = topology.plan_topology(["amd", "nvidia", "amd", "nvidia"])
    assert [i.ranks for i in layout.islands] == [(0, 2), (1, 3)]
    assert layout.bridge_ranks == (0, 1) and layout.needs_bridge
    assert layout.island_of(3).vendor == "nvidia" and layout.island_index(3) == 1
    sub = topology.plan_topology(["nvidia", "amd"], ranks=(1, 6))
    assert sub.members == (1, 6) and sub.index(6) == 1 and sub.island_of(6).leader == 6
    with pytest.raises(ValueError):
        topology.plan_topology([])
    with pytest.raises(ValueError, match="ascending"):
        topology.plan_topology(["amd", "amd"], ranks=(3, 1))
    assert not topology.plan_topology(["amd"] * 3).needs_bridge


def _peer(**kw):
    probe = Probe("nvidia", "2.11.0+cu128", "12.8", None, 1, True, True)
    base = dict(vendor="nvidia", simulated=False, hostname="h", bridge="gloo", probe=probe)
    base.update(kw)
    return topology.PeerInfo(**base)


def test_peer_wire_round_trip_keeps_reference_fields():
    wire = _peer(problems=("x",), policy_settings={"chunk_bytes": 8}).to_wire()
    for field in ("vendor", "simulated", "hostname", "bridge", "probe", "problems", "split_test",
                  "policy", "policy_settings", "gpu", "pinned_staging", "bridge_compression"):
        assert field in wire
    assert json.loads(json.dumps(wire)) == json.loads(json.dumps(wire))
    back = topology.PeerInfo.from_wire(json.loads(json.dumps(wire)))
    assert back == _peer(problems=("x",), policy_settings={"chunk_bytes": 8})
    # a dictionary with only the reference's fields still parses
    for extra in ("islands", "codec_format", "fabric", "pid"):
        wire.pop(extra)
    assert topology.PeerInfo.from_wire(wire).codec_format == "ref"


def test_validate_peers():
    topology.validate_peers([_peer(), _peer()])
    with pytest.raises(RuntimeError, match="1 of 2 ranks reported problems"):
        topology.validate_peers([_peer(), _peer(problems=("no GPU",))])
    with pytest.raises(RuntimeError, match="where to run"):
        topology.validate_peers([_peer(), _peer(simulated=True)])
    with pytest.raises(RuntimeError, match="different bridge transports"):
        topology.validate_peers([_peer(), _peer(bridge="nvlink")])
    with pytest.raises(RuntimeError, match="different collective policies"):
        topology.validate_peers([_peer(), _peer(policy="flat-gloo")])
    with pytest.raises(RuntimeError, match="settings of collective policy"):
        topology.validate_peers([_peer(policy_settings={"chunk_bytes": 8}), _peer()])
    with pytest.raises(RuntimeError, match="GPUBRIDGE_SPLIT_TEST"):
        topology.validate_peers([_peer(split_test="half"), _peer()])
    with pytest.raises(RuntimeError, match="GPUBRIDGE_PINNED_STAGING"):
        topology.validate_peers([_peer(pinned_staging=True), _peer()])
    with pytest.raises(RuntimeError, match="GPUBRIDGE_BRIDGE_COMPRESSION"):
        topology.validate_peers([_peer(bridge_compression="fp8"), _peer()])
    other = Probe("nvidia", "2.9.1+cu128", "12.8", None, 1, True, True)
    with pytest.warns(UserWarning, match="different PyTorch releases"):
        topology.validate_peers([_peer(), _peer(probe=other)])


def test_gpu_clashes():
    layout = topology.plan_topology(["nvidia", "nvidia", "amd", "amd"])
    hosts = ["h"] * 4
    assert topology.gpu_clashes(layout, hosts, ["g0", "g1", "g0", "g1"]) == []
    lines = topology.gpu_clashes(layout, hosts, ["g0", "g0", "g1", "g2"])
    assert len(lines) == 1 and "ranks [0, 1]" in lines[0]
    assert topology.gpu_clashes(layout, hosts, ["", "g0", "g1", "g1"])[0].startswith("  island 'amd'")
    assert topology.unchecked_islands(layout, ["", "g0", "g1", "g2"]) == ["  island 'nvidia': ranks [0]"]


def test_policy_registry_and_choice():
    two = topology.plan_topology(["nvidia", "amd"])
    one = topology.plan_topology(["nvidia", "nvidia"])
    assert policies.choose_policy("auto", two) is policies.ReduceBridgeBroadcast
    assert policies.choose_policy("auto", one) is policies.NativeOnly
    with pytest.raises(RuntimeError, match="doesn't apply"):
        policies.choose_policy(policies.ShardedBridge, one)
    with pytest.raises(ValueError, match="unknown collective policy"):
        policies.resolve_policy("fastest")
    with pytest.raises(TypeError):
        policies.resolve_policy(3)

    class Mine(policies.FlatGloo):
        name = "mine"
    assert policies.register_policy(Mine) is Mine and policies.resolve_policy("mine") is Mine

    class Clash(policies.FlatGloo):
        name = "mine"
    with pytest.raises(ValueError, match="already registered"):
        policies.register_policy(Clash)

    class Auto(policies.FlatGloo):
        name = "auto"
    with pytest.raises(ValueError, match="reserved"):
        policies.register_policy(Auto)
    assert not policies.implements(type("P", (policies.CollectivePolicy,), {}), "reduce_scatter_tensor")
    assert "flat-gloo" in policies.policies_implementing("all_gather_into_tensor", one)
    policies._POLICIES.pop("mine")


def test_thresholds_file(tmp_path, monkeypatch):
    path = tmp_path / "t.json"
    rules = [{"max_bytes": 65536, "policy": "flat-gloo"},
             {"max_bytes": None, "policy": "pipelined-reduce-bridge-broadcast"}]
    policies.write_thresholds(str(path), rules, 1 << 20)
    assert policies.load_thresholds(str(path), 4 << 20) == {"rules": rules, "chunk_bytes": 1 << 20}
    monkeypatch.setenv(config.THRESHOLDS_ENV, str(path))
    assert policies.AutoTuned.settings()["rules"] == rules
    for broken, message in [
        ({"rules": rules}, "not a gpubridge thresholds file"),
        ({"gpubridge_thresholds": 1, "rules": []}, "non-empty list"),
        ({"gpubridge_thresholds": 1, "rules": [{"max_bytes": None, "policy": "nope"}]}, "names policy"),
        ({"gpubridge_thresholds": 1, "rules": [{"max_bytes": 5, "policy": "auto"}]}, "last rule"),
        ({"gpubridge_thresholds": 1, "rules": [{"max_bytes": 9, "policy": "auto"},
                                               {"max_bytes": 4, "policy": "auto"},
                                               {"max_bytes": None, "policy": "auto"}]}, "larger than"),
        ({"gpubridge_thresholds": 1, "rules": rules, "chunk_bytes": 12}, "multiple of 8"),
    ]:
        path.write_text(json.dumps(broken))
        with pytest.raises(ValueError, match=message):
            policies.load_thresholds(str(path), 4 << 20)
    path.write_text("{not json")
    with pytest.raises(ValueError, match="not valid JSON"):
        policies.load_thresholds(str(path), 8)
    with pytest.raises(ValueError, match="can't read it"):
        policies.load_thresholds(str(tmp_path / "missing.json"), 8)


def test_transport_registry():
    assert transport.resolve_transport("gloo") is transport.GlooTransport
    assert transport.resolve_transport("nvlink").device_tensors
    with pytest.raises(ValueError, match="unknown bridge transport"):
        transport.resolve_transport("carrier-pigeon")
    with pytest.raises(ValueError, match="can't be loaded"):
        transport.resolve_transport("ucx")
    with pytest.raises(TypeError):
        transport.register_transport(int)


def test_compression_kernel_setting_and_multitcp_interface(monkeypatch):
    from gpubridge_b200 import compression as C
    from gpubridge_b200 import multitcp
    import torch
    monkeypatch.setenv("GPUBRIDGE_COMPRESSION_KERNELS", "torch")
    assert C.kernels_setting() == "torch" and C._device_codec(torch.zeros(1)) is None
    monkeypatch.setenv("GPUBRIDGE_COMPRESSION_KERNELS", "triton")
    assert C.kernels_setting() == "native"
    import pytest
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        C._device_codec(torch.zeros(1))
    monkeypatch.setenv("GPUBRIDGE_COMPRESSION_KERNELS", "sometimes")
    with pytest.raises(ValueError):
        C.kernels_setting()
    monkeypatch.delenv("GPUBRIDGE_COMPRESSION_KERNELS")
    monkeypatch.delenv("GPUBRIDGE_MULTITCP_IFADDR", raising=False)
    monkeypatch.setenv("GPUBRIDGE_MULTITCP_IFNAME", "lo")
    assert multitcp.listen_address().startswith("127.")
    monkeypatch.setenv("GPUBRIDGE_MULTITCP_IFNAME", "no-such-interface0")
    with pytest.raises(ValueError, match="no such interface"):
        multitcp.listen_address()
    monkeypatch.setenv("GPUBRIDGE_MULTITCP_IFADDR", "10.1.2.3")
    assert multitcp.listen_address() == "10.1.2.3"


def test_utils_clock_summary_and_timing():
    import torch
    from gpubridge_b200.utils import clocks, device_time, human_bytes, max_over_ranks
    lines = ["0, 1920, 1965, 650.1, 0x0000000000000004, Not Active, Not Active, Not Active, Active",
             "0, 1350, 1965, 990.0, 0x0000000000000004, Not Active, Not Active, Not Active, Active",
             "garbage", "0, 1400, 1965, 991.0, 0x0, Not Active, Active, Not Active, Not Active"]
    s = clocks.summarise(lines)
    assert s["sm_mhz"] == 1400 and s["sm_max_mhz"] == 1965 and s["samples"] == 3
    assert s["reasons"] == ["hw_thermal_slowdown", "sw_power_cap"] and not clocks.acceptable(s)
    assert clocks.acceptable(clocks.summarise(lines[:2]))                    # a power cap is kept
    assert not clocks.acceptable({"sm_mhz": 600.0, "sm_max_mhz": 1965.0, "reasons": []})
    calls = []
    ms = device_time(lambda n: calls.append(n), 7, torch.device("cpu"), barrier=lambda: calls.append("b"))
    assert calls == ["b", 7, "b"] and ms >= 0
    assert max_over_ranks(3.5) == 3.5 and human_bytes(4 << 20) == "4M" and human_bytes(1000) == "1000"


def test_shards_cover_every_file_once():
    from conftest import shard_of
    files = [f"tests/test_{i}.py" for i in range(11)]
    shards = [shard_of(files, f"{k}/4") for k in range(1, 5)]
    assert set().union(*shards) == set(files) and sum(len(s) for s in shards) == len(files)
    assert max(len(s) for s in shards) - min(len(s) for s in shards) <= 1
    import pytest
    with pytest.raises(ValueError):
        shard_of(files, "5/4")


def test_link_layout_from_a_fake_nvml():
    from gpubridge_b200.utils.links import link_layout

    class FakeNvml:
        NVML_NVLINK_MAX_LINKS = 18

        def __init__(self, links, remote, broken=()):
            self.links, self.remote, self.broken, self.calls = links, remote, broken, []

        def nvmlInit(self): self.calls.append("init")
        def nvmlShutdown(self): self.calls.append("shutdown")
        def nvmlDeviceGetCount(self): return len(self.links)
        def nvmlDeviceGetHandleByIndex(self, i): return i
        def nvmlDeviceGetName(self, h): return b"NVIDIA B200"

        def nvmlDeviceGetNvLinkState(self, h, link):
            if link >= 18 - len(self.broken) and h in self.broken:
                raise RuntimeError("not supported")
            return 1 if link < self.links[h] else 0

        def nvmlDeviceGetNvLinkVersion(self, h, link): return 5
        def nvmlDeviceGetNvLinkRemoteDeviceType(self, h, link): return self.remote

    box = FakeNvml([18] * 8, remote=2)
    layout = link_layout(box)
    assert layout["fabric"] == "nvswitch" and not layout["links_uneven"]
    assert layout["gpus"][3] == {"index": 3, "name": "NVIDIA B200", "links_active": 18, "link_version": 5,
                                 "to_switch": 18, "to_gpu": 0, "to_other": 0}
    assert box.calls == ["init", "shutdown"]                 # only getters in between
    assert link_layout(FakeNvml([4, 4], remote=0))["fabric"] == "direct"
    lost = link_layout(FakeNvml([18, 16], remote=2))
    assert lost["links_uneven"] and lost["fabric"] == "nvswitch"
    assert link_layout(FakeNvml([0, 0], remote=2))["fabric"] == "none"

    class NoNvml:
        def nvmlInit(self): raise OSError("libnvidia-ml.so not found")

    assert link_layout(NoNvml()) is None
