"""bench.py's outer logic without a GPU: a team whose in-switch path fails measures once more on
the peer-memory kernels (the process re-executes itself with the switch off, once), a lone rank
and a second failure raise, and the reference arm reports instead of raising."""
import importlib.util
import json
import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


@pytest.fixture
def bench(monkeypatch):
    spec = importlib.util.spec_from_file_location("bench_under_test", ROOT / "bench.py")
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    for name in ("GPUBRIDGE_NVLS", "GPUBRIDGE_BENCH_SECOND_TRY"):
        monkeypatch.delenv(name, raising=False)
    monkeypatch.setenv("RANK", "0")
    monkeypatch.setenv("LOCAL_RANK", "0")
    monkeypatch.setattr(sys, "argv", ["bench.py", "--gpus", "4", "--steps", "5", "--warmup", "3"])
    return module


def _boom(args):
    raise RuntimeError("a wait inside a kernel ran out")


def test_a_team_tries_once_more_without_the_switch(bench, monkeypatch):
    monkeypatch.setenv("WORLD_SIZE", "4")
    monkeypatch.setattr(bench, "run_ours", _boom)
    calls = []
    monkeypatch.setattr(os, "execv", lambda exe, argv: calls.append((exe, argv, dict(os.environ))))
    with pytest.raises(RuntimeError):               # only because the stand-in for execv returns
        bench.main()
    (exe, argv, env), = calls
    assert exe == sys.executable and argv[1:] == sys.argv
    assert env["GPUBRIDGE_NVLS"] == "0" and env["GPUBRIDGE_BENCH_SECOND_TRY"] == "1"


def test_the_second_failure_and_a_lone_rank_raise(bench, monkeypatch):
    monkeypatch.setattr(bench, "run_ours", _boom)
    monkeypatch.setattr(os, "execv", lambda *a: pytest.fail("must not re-execute"))
    monkeypatch.setenv("WORLD_SIZE", "4")
    monkeypatch.setenv("GPUBRIDGE_BENCH_SECOND_TRY", "1")
    with pytest.raises(RuntimeError):
        bench.main()
    monkeypatch.delenv("GPUBRIDGE_BENCH_SECOND_TRY")
    monkeypatch.setenv("WORLD_SIZE", "1")
    with pytest.raises(RuntimeError):
        bench.main()


def test_the_second_try_says_so_and_the_reference_arm_reports(bench, monkeypatch, capsys):
    monkeypatch.setenv("WORLD_SIZE", "4")
    monkeypatch.setenv("GPUBRIDGE_BENCH_SECOND_TRY", "1")
    monkeypatch.setattr(bench, "run_ours", lambda args: {"value": 1.0, "config": {"model": "x"}})
    bench.main()
    line = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert line["config"]["second_try_without_in_switch_reduction"] is True
    monkeypatch.setattr(sys, "argv", ["bench.py", "--impl", "reference", "--gpus", "4"])
    monkeypatch.setattr(bench, "run_reference", _boom)
    bench.main()
    line = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert line["impl"] == "reference" and "ran out" in line["unavailable"]
