"""The node report of the kit against a pretend /sys, /proc, /boot and /etc: what it reads, what it
says when something is missing, and that it never fails."""
import json
import platform

from gpubridge_b200.kit import node_report


def _tree(tmp_path):
    root = tmp_path / "root"
    port = root / "sys" / "class" / "infiniband" / "mlx5_0" / "ports" / "1"
    port.mkdir(parents=True)
    (port / "state").write_text("4: ACTIVE\n")
    (port / "rate").write_text("400 Gb/sec (4X NDR)\n")
    (port / "link_layer").write_text("InfiniBand\n")
    (root / "sys" / "class" / "infiniband" / "mlx5_0" / "fw_ver").write_text("28.39.1002\n")
    nic = root / "sys" / "class" / "net" / "eth0"
    nic.mkdir(parents=True)
    (nic / "operstate").write_text("up\n")
    (nic / "mtu").write_text("9000\n")
    (nic / "speed").write_text("100000\n")
    (root / "proc").mkdir()
    (root / "proc" / "modules").write_text("nvidia 1 2 - Live 0x0\nmlx5_core 3 4 - Live 0x0\nsnd 5 6 - Live 0x0\n")
    (root / "boot").mkdir()
    (root / "boot" / f"config-{platform.release()}").write_text(
        "CONFIG_PCI_P2PDMA=y\n# CONFIG_DMABUF_MOVE_NOTIFY is not set\nCONFIG_OTHER=y\n")
    (root / "etc").mkdir()
    (root / "etc" / "os-release").write_text('PRETTY_NAME="Pretend Linux 1"\n')
    return root


def test_reads_the_pretend_node(tmp_path):
    facts = node_report.report(_tree(tmp_path), find_library=lambda name: None)
    assert facts["kernel"]["distribution"] == "Pretend Linux 1"
    assert facts["kernel"]["config"] == {"CONFIG_PCI_P2PDMA": "y", "CONFIG_DMABUF_MOVE_NOTIFY": "not set"}
    assert set(facts["modules"]["loaded"]) == {"nvidia", "mlx5_core"} and "nvidia_peermem" in facts["modules"]["missing"]
    port = facts["rdma"]["devices"]["mlx5_0"]["ports"]["1"]
    assert port["state"] == "4: ACTIVE" and port["link_layer"] == "InfiniBand"
    assert facts["rdma"]["libibverbs"] is None and facts["rdma"]["ibv_reg_dmabuf_mr"] is None
    assert facts["net"]["interfaces"]["eth0"] == {"state": "up", "mtu": "9000", "speed_mbps": 100000, "address": None}
    assert facts["ucx"]["libucp"] is None


def test_an_empty_node_leaves_notes_not_errors(tmp_path):
    out = tmp_path / "out"
    assert node_report.main([str(out), "--root", str(tmp_path / "nothing")]) == 0
    told = json.loads((out / "report.json").read_text())
    assert told["rdma"]["devices"] == {} and told["modules"]["loaded"] == {}
    assert "not found on this node" in (out / "rdma.txt").read_text()
    assert {p.name for p in out.iterdir()} >= {"kernel.txt", "modules.txt", "rdma.txt", "net.txt", "gpus.txt",
                                                 "ucx.txt", "report.json"}


def test_a_subject_that_blows_up_is_reported_not_raised(tmp_path, monkeypatch):
    monkeypatch.setattr(node_report, "net", lambda root: 1 / 0)
    facts = node_report.report(tmp_path)
    assert "ZeroDivisionError" in facts["net"]["error"] and "kernel" in facts
