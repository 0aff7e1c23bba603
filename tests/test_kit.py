"""The validation kit on CPU ranks: the thirteen-stage check and its summary, the negative
init test, the point-to-point checks through the torch backend, and redaction."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _torchrun(nproc, port, module, *args, env=None, timeout=300):
    full = dict(os.environ, PYTHONPATH=ROOT, OMP_NUM_THREADS="1", **(env or {}))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1",
           f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1", "--master-port", str(port),
           "-m", module, *args]
    return subprocess.run(cmd, env=full, cwd=ROOT, capture_output=True, text=True,
                          timeout=timeout)


SIM = {"GPUBRIDGE_VENDOR": "nvidia", "GPUBRIDGE_SPLIT_TEST": "half"}


def test_check_and_summary(tmp_path):
    out = tmp_path / "check"
    done = _torchrun(2, 29721, "gpubridge_b200.kit.check", "--out", str(out),
                     "--in-flight-settle", "0.2", "--timeout", "120", env=SIM)
    assert done.returncode == 0, done.stderr[-3000:]
    from gpubridge_b200.kit import summarize
    assert summarize.main([str(out)]) == 0
    summary = json.loads((out / "summary.json").read_text())
    assert summary["ok"] and summary["split_test"] == "half"
    assert list(summary["stages"]) == [
        "init", "device", "dtypes", "busy_gpu", "broadcast", "reductions", "all_gather",
        "reduce_scatter", "async", "reduction_agreement", "in_flight", "barrier", "destroy"]
    assert "SPLIT TEST" in (out / "summary.md").read_text()
    # a missing rank fails the summary unless it is declared partial
    (out / "rank1.json").unlink()
    assert summarize.main([str(out)]) == 1
    assert summarize.main(["--partial", str(out)]) == 0


def test_expected_init_error(tmp_path):
    out = tmp_path / "neg"
    done = _torchrun(2, 29722, "gpubridge_b200.kit.check", "--out", str(out),
                     "--expect-init-error", "No GPU is visible", "--timeout", "60",
                     env={"GPUBRIDGE_VENDOR": ""})
    assert done.returncode == 0, done.stderr[-3000:]
    record = json.loads((out / "rank0.json").read_text())
    assert record["ok"] and record["stages"][0]["name"] == "expected_init_error"
    # the wrong pattern fails the run
    done = _torchrun(2, 29723, "gpubridge_b200.kit.check", "--out", str(tmp_path / "neg2"),
                     "--expect-init-error", "LOCAL_RANK", "--timeout", "60",
                     env={"GPUBRIDGE_VENDOR": ""})
    assert done.returncode != 0


def test_p2p_only(tmp_path):
    out = tmp_path / "p2p"
    done = _torchrun(2, 29724, "gpubridge_b200.kit.check", "--out", str(out), "--p2p-only",
                     "--timeout", "120", env=SIM)
    assert done.returncode == 0, done.stderr[-3000:]
    record = json.loads((out / "rank1.json").read_text())
    cases = record["stages"][1]["cases"]
    assert len(cases) == 30 and all(c["ok"] for c in cases)


def test_redaction(monkeypatch, tmp_path):
    from gpubridge_b200 import kit
    monkeypatch.setenv("HOME", "/home/somebody")
    text = kit.redact("see /home/somebody/run and https://me:secret@host/x")
    assert "somebody" not in text and "secret" not in text and "~/run" in text
    env = kit.recorded_env({"GPUBRIDGE_POLICY": "auto", "GPUBRIDGE_API_TOKEN": "x",
                            "HOME": "/h", "NCCL_DEBUG": "INFO"})
    assert env == {"GPUBRIDGE_POLICY": "auto", "NCCL_DEBUG": "INFO"}
    kit.write_json(tmp_path / "a" / "b.json", {"p": "/home/somebody/x", "n": [1, {"q": (2,)}]})
    assert json.loads((tmp_path / "a" / "b.json").read_text()) == {"p": "~/x", "n": [1, {"q": [2]}]}


def test_numerical_gate_software_only(tmp_path):
    """The bridged arm passes its positive runs and every negative control fails."""
    out = tmp_path / "gate"
    done = _torchrun(4, 29725, "gpubridge_b200.kit.numerical_gate", "--software-only",
                     "--out", str(out), "--timeout", "120")
    assert done.returncode == 0, done.stderr[-3000:]
    result = json.loads((out / "gate.json").read_text())
    assert result["passed"] and "bridged/sgd/sum" in result["runs"]
    from gpubridge_b200.kit import numerical_gate as gate
    records = []
    for r in range(4):
        records += json.loads((out / f"gate-bridged-rank{r}.json").read_text())
    # a control that passes, or a positive run that fails, flips the verdict
    broken = [dict(r, passed=True) if r["control"] == "scale" else r for r in records]
    assert not gate.verdict(broken)["passed"]
    broken = [dict(r, passed=False) if r["control"] == "none" and r["rank"] == 2 else r
              for r in records]
    assert not gate.verdict(broken)["passed"]


def test_preflight_two_sides_on_one_machine(tmp_path):
    """Master and worker on this machine: interfaces listed, a pair chosen both ways, the Gloo
    check passes, both records written."""
    env = dict(os.environ, PYTHONPATH=ROOT)
    base = [sys.executable, "-m", "gpubridge_b200.kit.preflight", "--master-addr", "127.0.0.1",
            "--port", "29726", "--bandwidth-seconds", "0.2", "--out", str(tmp_path)]
    master = subprocess.Popen(base + ["--role", "master"], env=env, cwd=ROOT,
                              stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
    worker = subprocess.run(base + ["--role", "worker"], env=env, cwd=ROOT, capture_output=True,
                            text=True, timeout=120)
    out, err = master.communicate(timeout=120)
    assert worker.returncode == 0, worker.stderr[-2000:]
    assert master.returncode == 0, err[-2000:]
    for role in ("master", "worker"):
        record = json.loads((tmp_path / f"preflight-{role}.json").read_text())
        assert record["ok"] and record["checks"]["gloo"] == "ok"
        assert record["chosen_ifname"] and record["bandwidth"]["out_MBps"] > 0


def test_probe_without_gpu(tmp_path):
    from gpubridge_b200.kit import probe
    import torch
    if torch.cuda.is_available():
        pytest.skip("the CPU form of the probe")
    assert probe.main(["--out", str(tmp_path), "--allow-no-gpu"]) == 0
    assert probe.main(["--out", str(tmp_path / "strict")]) == 1       # no GPU is a failure by default
    record = json.loads((tmp_path / "strict" / "probe.json").read_text())
    assert record["stages"][0]["name"] == "gpus_visible" and record["stages"][0]["ok"] is False


def test_runbook_plan_and_one_step(tmp_path):
    from gpubridge_b200.kit import runbook
    steps = runbook.plan(tmp_path, 8, cpu=False)
    names = [s["name"] for s in steps]
    assert names[0] == "probe" and "check-3+5" in names and "streams" in names
    assert "gate-bridged" in names and "scaling-8" in names and names[-1] == "scaling-summary"
    assert runbook.main(["--out", str(tmp_path), "--gpus", "2", "--cpu", "--dry-run"]) == 0
    # one real step, and a failing one is recorded without stopping the run
    os.environ["GPUBRIDGE_VENDOR"] = "nvidia"
    try:
        assert runbook.main(["--out", str(tmp_path / "run"), "--gpus", "2", "--cpu", "--only", "probe"]) == 0
    finally:
        os.environ.pop("GPUBRIDGE_VENDOR", None)
    rows = [json.loads(l) for l in (tmp_path / "run" / "steps.jsonl").read_text().splitlines()]
    assert rows == [dict(rows[0], step="probe", ok=True)]
    bad = runbook.run_step({"name": "boom", "cmd": [sys.executable, "-c", "raise SystemExit(3)"],
                            "env": {}, "expect": None, "timeout": None}, tmp_path / "run", 30)
    assert bad["ok"] is False and bad["exit_code"] == 3


def test_triage_puts_problems_first(tmp_path, capsys):
    """A fabricated runbook directory: a failed step, a step past its limit, a log without a
    verdict and a failed check summary all appear above the detail; addresses are redacted."""
    import tarfile
    from gpubridge_b200.kit import triage

    run = tmp_path / "rb"
    (run / "check-half").mkdir(parents=True)
    (run / "probe").mkdir()
    rows = [{"step": "probe", "ok": True, "exit_code": 0, "seconds": 1.0, "log": "probe.log"},
            {"step": "sweep", "ok": False, "exit_code": 1, "seconds": 3.0, "log": "sweep.log"},
            {"step": "sweep", "ok": False, "exit_code": 2, "seconds": 4.0, "log": "sweep.log"},
            {"step": "gate-bridged", "ok": False, "exit_code": None, "seconds": 9.0, "log": "gate-bridged.log"}]
    (run / "steps.jsonl").write_text("\n".join(json.dumps(r) for r in rows) + "\n")
    (run / "probe.log").write_text("fine\n")
    (run / "sweep.log").write_text("starting\nRuntimeError: connect to 10.1.2.3 refused by node-17\nbye\n")
    (run / "gate-bridged.log").write_text("the step ran past its limit\n")
    (run / "p2p.log").write_text("half a line")
    (run / "check-half" / "summary.json").write_text(json.dumps(
        {"ok": False, "stages": {"init": {"0": True, "1": True}, "all_reduce": {"0": True, "1": False}},
         "ranks_missing": []}))
    (run / "probe" / "probe.json").write_text(json.dumps(
        {"environment": {"hostname": "node-17", "device_count": 2, "devices": [{"name": "B200"}, {"name": "B200"}],
                         "torch": "2.11", "torch_cuda": "12.8", "nccl": "2.28.9", "gpubridge_b200": "0.1.0"}}))
    (run / "sweep.json").write_text(json.dumps(
        [{"bytes": 1 << 20, "target": "ours", "ms": 0.02, "busbw_gbs": 90.0},
         {"bytes": 1 << 20, "target": "nccl", "ms": 0.03, "busbw_gbs": 60.0}]))

    assert triage.main([str(run)]) == 1
    text = capsys.readouterr().out
    assert text.index("PROBLEMS") < text.index("ran on host 1")
    assert "step sweep: FAILED (exit code 2" in text and "exit code 1" not in text
    assert "step gate-bridged: FAILED (ran past its limit" in text
    assert "step p2p: left unfinished" in text
    assert "check-half: all_reduce: r1" in text
    assert "10.1.2.3" not in text and "node-17" not in text and "<ip>" in text
    assert "ours = 1.50x nccl's speed" in text
    assert "verdict: 0 of 1 run(s) clean" in text

    ball = tmp_path / "rb.tgz"
    with tarfile.open(ball, "w:gz") as tar:
        tar.add(run, arcname="results/rb")
    assert triage.main([str(ball), "--max-lines", "6"]) == 1
    short = capsys.readouterr().out.splitlines()
    assert len(short) == 6 and short[-1].startswith("verdict") and "more lines" in short[-2]
    (tmp_path / "empty").mkdir()
    assert triage.main([str(tmp_path / "empty")]) == 2


def test_validation_tables_never_count_simulation(tmp_path, capsys):
    """Two fabricated jobs: a CPU-simulation job that passed everything and a GPU job with one
    failed stage.  Items the simulation alone covers read "simulation only"; the GPU job's
    failure makes its item FAILED; hosts are numbered."""
    from gpubridge_b200.kit import validation_tables

    def job(name, cuda, bad_stage=None, extra_steps=()):
        d = tmp_path / "results" / name
        (d / "check-half").mkdir(parents=True)
        (d / "probe").mkdir()
        env = {"hostname": f"secret-{name}", "cuda_available": cuda, "device_count": 8 if cuda else 0,
               "devices": [{"name": "NVIDIA B200"}] * (8 if cuda else 0), "torch": "2.11", "torch_cuda": "12.8",
               "nccl": "2.28.9", "gpubridge_b200": "0.1.0", "env": {} if cuda else {"GPUBRIDGE_VENDOR": "nvidia"}}
        rows = [{"step": s, "ok": True, "exit_code": 0, "seconds": 1, "log": f"{s}.log"}
                for s in ("probe", "check-half", "summary-half", "sweep", *extra_steps)]
        (d / "steps.jsonl").write_text("\n".join(json.dumps(r) for r in rows) + "\n")
        stages = {s: {"0": True, "1": s != bad_stage} for s in ("init", "device", "dtypes", "broadcast", "barrier", "destroy")}
        (d / "check-half" / "summary.json").write_text(json.dumps({"ok": bad_stage is None, "stages": stages, "ranks_missing": []}))
        (d / "check-half" / "rank0.json").write_text(json.dumps({"environment": env}))
        (d / "probe" / "probe.json").write_text(json.dumps({"environment": env}))
        (d / "sweep.json").write_text(json.dumps([{"bytes": 1 << 20, "target": "ours", "ms": 0.02, "busbw_gbs": 90.0},
                                                  {"bytes": 1 << 20, "target": "nccl", "ms": 0.03, "busbw_gbs": 60.0}]))

    job("sim", cuda=False, extra_steps=("p2p",))
    job("gpu", cuda=True, bad_stage="dtypes")
    assert validation_tables.main([str(tmp_path / "results")]) == 1
    text = capsys.readouterr().out
    assert "secret" not in text and "host 1" in text and "host 2" in text
    assert "| sim | CPU simulation | 5 |" in text and "| gpu | GPU | 4 |" in text and "8 x NVIDIA B200" in text
    data = json.loads((tmp_path / "results" / "validation_tables.json").read_text())
    verdicts = {i["item"]: i["verdict"] for i in data["items"]}
    assert verdicts["dtypes"] == "FAILED" and verdicts["discovery"] == "passed"
    assert verdicts["p2p"] == "simulation only" and verdicts["numerics"] == "not run"
    assert {(b["job"], b["speed_vs_nccl"]) for b in data["benchmarks"]} == {("sim", 1.5), ("gpu", 1.5)}
