"""The kit programs of the RDMA-style endpoint run end to end on the in-process fabric."""
import json

import pytest

from gpubridge_b200.kit import rdma_kit
from gpubridge_b200.ops import _lib

pytestmark = pytest.mark.skipif(not _lib.available(), reason="the native library is not built")


def test_check_passes_every_scenario_and_records_them(tmp_path):
    assert rdma_kit.main(["check", "--out", str(tmp_path)]) == 0
    rows = json.loads((tmp_path / "rdma_check.json").read_text())["rows"]
    names = [r["scenario"] for r in rows]
    assert "rendezvous message" in names and "fault: kill" in names and len(rows) >= 17
    assert sum(name.startswith("device registration") for name in names) == 3
    assert all(r["ok"] for r in rows)
    kill = next(r for r in rows if r["scenario"] == "fault: kill")
    assert any(kill["members_failed"]) and kill["seconds"] < 10


def test_perf_and_ab_write_their_tables(tmp_path):
    assert rdma_kit.main(["perf", "--out", str(tmp_path), "--trials", "3", "--sizes", "64,262144"]) == 0
    perf = json.loads((tmp_path / "rdma_perf.json").read_text())["rows"]
    assert [r["bytes"] for r in perf] == [64, 262144] and all(r["one_way_us"] > 0 for r in perf)
    assert rdma_kit.main(["ab", "--out", str(tmp_path), "--trials", "2", "--numel", str(1 << 16)]) == 0
    ab = json.loads((tmp_path / "rdma_ab.json").read_text())["rows"]
    assert len(ab) == len(rdma_kit.ARMS) and ab[0]["against_first"] == 1.0
    assert all(r["routes"] == {"bounce": 3} for r in ab)


def test_perf_over_the_socket_provider(tmp_path):
    assert rdma_kit.main(["perf", "--out", str(tmp_path), "--trials", "2", "--sizes", "64,100000",
                          "--fabric", "sockets"]) == 0
    rows = json.loads((tmp_path / "rdma_perf.json").read_text())["rows"]
    assert [r["fabric"] for r in rows] == ["sockets", "sockets"] and all(r["one_way_us"] > 0 for r in rows)
