"""The kit's building blocks one by one, in this process: journals and their summaries (missing
ranks, partial summaries, a rank left inside a stage, a GPU shared by mistake, the split-test
banner, weak-scaling efficiency), what a record may contain (allow-listed variables, no secrets,
redacted paths and credentials), the stream-mutation audit's verdicts from JUnit reports, the
baseline identity's digests, the report helpers and the preflight's interface choice.
(Reference: the helper-level cases of tests/test_gpu_kit.py.)"""
import json
import os
import sys
from pathlib import Path

import pytest
import torch

from gpubridge_b200 import kit
from gpubridge_b200.kit import baseline_identity, preflight, probe, report, stream_mutations, summarize


# ---- journals -----------------------------------------------------------------------------------------
def journal(tmp_path, rank, world=2, stages=(("init", True), ("all_reduce", True)), split=None, ok=None,
            device="cpu", bus=None, host="box"):
    data = {"kit_version": 1, "program": "check", "ok": all(s[1] for s in stages) if ok is None else ok,
            "environment": {"torch": "2.x", "hostname": host,
                            "devices": [{"index": 0, "pci_bus_id": bus}] if bus else []},
            "run": {"kind": "gpu-split-test" if split else "cpu-simulation", "world_size": world, "rank": rank,
                    "split_test": split, "policy": "auto", "fused": False, "device": device,
                    "islands": [{"vendor": "nvidia", "ranks": list(range(world)), "leader": 0}]},
            "stages": [{"name": n, "ok": v, **({"error": f"{n} broke"} if v is False else {})} for n, v in stages]}
    (tmp_path / f"rank{rank}.json").write_text(json.dumps(data))


def test_a_journal_records_each_stage_and_the_stage_a_rank_died_in(tmp_path):
    record = kit.Journal(tmp_path / "rank0.json", "demo", hang_dump_seconds=0)
    with record.stage("first") as entry:
        entry["measured"] = 3
    on_disk = json.loads((tmp_path / "rank0.json").read_text())
    assert on_disk["stages"] == [{"name": "first", "ok": True, "measured": 3, "seconds": on_disk["stages"][0]["seconds"]}]
    assert on_disk["ok"] is None                                   # not closed yet: the run is still going
    with pytest.raises(ZeroDivisionError):
        with record.stage("second"):
            # while a stage runs, the file says so: that is what a hung rank leaves behind
            assert json.loads((tmp_path / "rank0.json").read_text())["stages"][1]["ok"] is None
            1 / 0
    with record.stage("third") as entry:
        entry["ok"] = False                                        # a stage may fail without raising
    assert record.close() == 1
    on_disk = json.loads((tmp_path / "rank0.json").read_text())
    assert [s["ok"] for s in on_disk["stages"]] == [True, False, False] and on_disk["ok"] is False
    assert "ZeroDivisionError" in on_disk["stages"][1]["error"] and "finished" in on_disk
    clean = kit.Journal(tmp_path / "rank1.json", "demo", hang_dump_seconds=0)
    with clean.stage("only"):
        pass
    assert clean.close() == 0


def test_summary_fails_on_missing_ranks_unless_partial(tmp_path):
    journal(tmp_path, 0, world=3)
    journal(tmp_path, 2, world=3)
    summary, text = summarize.summarize(tmp_path)
    assert not summary["ok"] and summary["ranks_missing"] == [1] and "Missing ranks" in text
    summary, text = summarize.summarize(tmp_path, partial=True)
    assert summary["ok"] and summary["ranks_missing"] == [1] and "another machine" in text
    assert summarize.summarize(tmp_path / "empty")[0]["ok"] is False


def test_summary_names_failed_stages_and_ranks_left_inside_one(tmp_path):
    journal(tmp_path, 0, stages=(("init", True), ("all_reduce", False)))
    journal(tmp_path, 1, stages=(("init", True), ("all_reduce", None)), ok=None)
    summary, text = summarize.summarize(tmp_path)
    assert not summary["ok"]
    assert summary["errors"] == {"rank 0 / all_reduce": "all_reduce broke",
                                 "rank 1 / all_reduce": "the rank was left inside this stage"}
    assert summary["stages"]["all_reduce"] == {0: False, 1: None}
    assert "| all_reduce | FAIL | - |" in text and text.startswith(f"# {tmp_path.name}: FAIL")


def test_summary_carries_the_split_test_banner(tmp_path):
    journal(tmp_path, 0, split="half")
    journal(tmp_path, 1, split="half")
    summary, text = summarize.summarize(tmp_path)
    assert summary["ok"] and summary["split_test"] == "half" and summarize.BANNER in text
    journal(tmp_path, 0)
    journal(tmp_path, 1)
    assert summarize.BANNER not in summarize.summarize(tmp_path)[1]


def test_summary_flags_a_shared_gpu_outside_a_split_test(tmp_path):
    journal(tmp_path, 0, device="cuda:0", bus="1b:00")
    journal(tmp_path, 1, device="cuda:0", bus="1b:00")
    summary, text = summarize.summarize(tmp_path)
    assert not summary["ok"] and "share one GPU" in summary["errors"]["ranks [0, 1]"]
    journal(tmp_path, 1, device="cuda:0", bus="1b:00", host="other-box")       # the same slot of another machine
    assert summarize.summarize(tmp_path)[0]["ok"]
    journal(tmp_path, 0, device="cuda:0", bus="1b:00", split="half")           # relabelling on purpose
    journal(tmp_path, 1, device="cuda:0", bus="1b:00", split="half")
    assert summarize.summarize(tmp_path)[0]["ok"]


def test_scaling_summary_computes_efficiency(tmp_path):
    for n, rate in ((1, 100.0), (2, 190.0), (4, 360.0)):
        (tmp_path / f"train-n{n}.json").write_text(json.dumps(
            {"world_size": n, "samples_per_sec": rate, "step_ms_median": 10.0, "params_in_sync": True}))
    summary, text = summarize.summarize_scaling(tmp_path)
    assert [round(r["efficiency"], 3) for r in summary["rows"]] == [1.0, 0.95, 0.9] and summary["ok"]
    assert "| 4 | 360.0 | 0.90 |" in text
    (tmp_path / "train-n8.json").write_text(json.dumps(
        {"world_size": 8, "samples_per_sec": 700.0, "params_in_sync": False}))
    assert not summarize.summarize_scaling(tmp_path)[0]["ok"]      # a run whose ranks drifted apart is no result
    assert summarize.main([str(tmp_path)]) in (0, 1) and (tmp_path / "summary.md").exists()
    assert summarize.main([]) == 2


# ---- what a record may contain ------------------------------------------------------------------------
def test_records_hold_only_allow_listed_variables_and_no_secrets():
    env = {"RANK": "3", "GPUBRIDGE_POLICY": "auto", "NCCL_DEBUG": "INFO", "KIT_TIMEOUT": "9",
           "GPUBRIDGE_API_TOKEN": "s3cret", "NCCL_SECRET_THING": "x", "AWS_SECRET_ACCESS_KEY": "y",
           "HOME": "/home/someone", "PATH": "/bin", "GPUBRIDGE_PASSWORD_FILE": "/p", "MASTER_ADDR": "10.0.0.1"}
    assert kit.recorded_env(env) == {"GPUBRIDGE_POLICY": "auto", "KIT_TIMEOUT": "9", "MASTER_ADDR": "10.0.0.1",
                                     "NCCL_DEBUG": "INFO", "RANK": "3"}


def test_redact_replaces_paths_users_and_url_credentials(monkeypatch):
    monkeypatch.setenv("HOME", "/home/ada")
    monkeypatch.setattr("getpass.getuser", lambda: "ada")
    assert kit.redact("clone https://ada:hunter2@example.org/r.git") == "clone https://***@example.org/r.git"
    assert kit.redact("/home/ada/work and /scratch/ada/x, not /home/adalbert") == "~/work and /scratch/$USER/x, not /home/adalbert"
    assert kit.scrub({"a": ["/home/ada", 3, {"b": "/scratch/ada"}], 4: None}) == {"a": ["~", 3, {"b": "/scratch/$USER"}], "4": None}
    monkeypatch.setattr("getpass.getuser", lambda: "root")
    assert kit.redact("/data/" + "root/x") == "/data/" + "root/x"   # the superuser's name is not worth hiding


def test_written_records_are_scrubbed_and_atomic(tmp_path, monkeypatch):
    monkeypatch.setenv("HOME", "/home/ada")
    monkeypatch.setattr("getpass.getuser", lambda: "ada")
    kit.write_json(tmp_path / "deep" / "r.json", {"where": Path("/home/ada/out"), "n": 1})
    assert json.loads((tmp_path / "deep" / "r.json").read_text()) == {"where": "~/out", "n": 1}
    assert not list((tmp_path / "deep").glob("*.tmp"))


def test_environment_names_versions_and_never_fails_without_a_gpu():
    told = kit.environment()
    for key in ("hostname", "python", "torch", "gpubridge_b200", "cuda_available", "device_count", "env", "probe"):
        assert key in told
    assert told["device_count"] == len(told["devices"])
    assert kit.default_timeout(7.0) == 7.0
    os.environ["KIT_TIMEOUT"] = "soon"
    try:
        assert kit.default_timeout(7.0) == 7.0
        os.environ["KIT_TIMEOUT"] = "12.5"
        assert kit.default_timeout(7.0) == 12.5
    finally:
        del os.environ["KIT_TIMEOUT"]
    import torch
    kit.queue_gpu_delay(torch.device("cpu"), 5.0)                  # nothing to delay on a CPU: returns at once
    kit.sync(torch.device("cpu"))


# ---- the stream-mutation audit ------------------------------------------------------------------------
JUNIT = """<testsuites><testsuite>
<testcase name="{a}">{a_body}</testcase>
<testcase name="other">{b_body}</testcase>
</testsuite></testsuites>"""


def verdict_of(tmp_path, switch, a_body="", b_body=""):
    run = stream_mutations.Run(switch, ["guard", "other"])
    report_file = tmp_path / "junit.xml"
    report_file.write_text(JUNIT.format(a="guard", a_body=a_body, b_body=b_body))
    run._read(report_file)
    return run


def test_each_mutation_names_an_existing_test_and_the_plan_has_one_control():
    table = stream_mutations.pairs()
    assert len(table) >= 3
    source = stream_mutations.TEST_FILE.read_text()
    for switch, test in table.items():
        assert f"def {test}(" in source, (switch, test)
    run = stream_mutations.Run("some-switch", ["test_a"])
    command = run.command("r.xml")
    assert command[:5] == [sys.executable, "-m", "pytest", "-m", "gpu"] and "--junitxml=r.xml" in command
    assert command[-1].endswith("test_gpu_streams.py::test_a")


def test_list_mode_prints_one_run_per_switch_and_one_without(capsys):
    assert stream_mutations.main(["--list"]) == 0
    lines = [line for line in capsys.readouterr().out.splitlines() if line.startswith("+ ")]
    table = stream_mutations.pairs()
    assert len(lines) == len(table) + 1
    assert sum(stream_mutations.SWITCH_ENV in line for line in lines) == len(table)
    one = sorted(table)[0]
    assert stream_mutations.main(["--list", "--mutation", one]) == 0
    assert len([line for line in capsys.readouterr().out.splitlines() if line.startswith("+ ")]) == 2


def test_the_audits_verdicts(tmp_path):
    wrong = '<failure message="AssertionError: 512 elements wrong after the copy">trace</failure>'
    crash = '<failure message="RuntimeError: CUDA error">trace</failure>'
    assert verdict_of(tmp_path, "s", wrong).verdict == "noticed"
    assert verdict_of(tmp_path, "s", wrong).good
    assert verdict_of(tmp_path, "s", crash).verdict == "failed for another reason"
    assert verdict_of(tmp_path, "s").verdict == "UNNOTICED" and not verdict_of(tmp_path, "s").good
    assert verdict_of(tmp_path, None).verdict == "clean run passes"
    assert verdict_of(tmp_path, None, wrong).verdict == "clean run FAILS"
    skipped = '<skipped message="needs a GPU"/>'
    assert verdict_of(tmp_path, "s", skipped, skipped).verdict == "did not run"
    assert verdict_of(tmp_path, None, '<error message="fixture failed">x</error>').verdict.startswith("broken")
    late = stream_mutations.Run("s", ["guard"])
    late.timed_out = True
    assert late.verdict == "timed out" and not late.good
    assert stream_mutations.Run("s", ["guard"]).verdict == "did not run"


# ---- identity, reports, preflight, probe ---------------------------------------------------------------
def test_tree_digests_see_content_and_names_but_not_build_output(tmp_path, monkeypatch):
    monkeypatch.setattr(baseline_identity, "ROOT", tmp_path)
    tree = tmp_path / "pkg"
    (tree / "sub").mkdir(parents=True)
    (tree / "a.py").write_text("x = 1\n")
    (tree / "sub" / "k.cu").write_text("__global__ void k() {}\n")
    first = baseline_identity.tree_digest(tree)
    assert first["files"] == 2
    (tree / "__pycache__").mkdir()
    (tree / "__pycache__" / "a.py").write_text("junk")
    (tree / "lib").mkdir()
    (tree / "lib" / "gen.py").write_text("junk")
    (tree / "notes.txt").write_text("not a source")
    assert baseline_identity.tree_digest(tree) == first
    (tree / "a.py").write_text("x = 2\n")
    changed = baseline_identity.tree_digest(tree)
    assert changed["sha256"] != first["sha256"]
    (tree / "a.py").rename(tree / "b.py")
    assert baseline_identity.tree_digest(tree)["sha256"] != changed["sha256"]       # a rename is a change
    assert baseline_identity.tree_digest(tmp_path / "absent") is None
    assert baseline_identity.tree_digest(tree / "b.py")["files"] == 1
    lib = tmp_path / "lib.so"
    lib.write_bytes(b"\x7fELF" + bytes(100))
    told = baseline_identity.library(lib)
    assert told["bytes"] == 104 and len(told["sha256"]) == 64 and baseline_identity.library(tmp_path / "no.so") is None
    assert baseline_identity.version_of("torch") and baseline_identity.version_of("no-such-package-xyz") is None
    assert baseline_identity.run("definitely-not-a-command") is None


def test_the_identity_record_has_every_part():
    record = baseline_identity.identity()
    assert set(record) == {"source", "native", "toolchain", "packages", "reference", "environment"}
    assert set(record["source"]["trees"]) == set(baseline_identity.TREES)
    assert record["source"]["trees"]["gpubridge_b200/csrc"]["files"] > 10
    assert record["packages"]["torch"] and "flags" in record["native"]


def test_report_helpers():
    assert report.curve_gaps([1.0, 2.0, 3.5], [1.0, 2.5, 3.0, 9.0], tail=2) == (0.5, 0.5)
    assert report.curve_gaps([5.0], [1.0], tail=10) == (4.0, 4.0)
    drawn = report.svg([("a", [3.0, 2.0, 1.0]), ("b", [3.0, 2.5, 2.0])])
    assert drawn.startswith("<svg") and drawn.count("<polyline") == 2 and "a" in drawn
    assert report.svg([("flat", [1.0, 1.0])]).startswith("<svg")   # a flat curve must not divide by zero
    assert report.label("x", {"mode": "hsdp", "world": 8, "compression": "fp8"}) == "x: hsdp x8 fp8"
    assert report.label("p", {"bench": "train_pipeline", "schedule": "1f1b", "stages": 4}) == "p: pipeline 1f1b x4"
    assert report.ddp_verdict({"params_in_sync": True}) == "no per-step check"
    assert "DIFFER" in report.ddp_verdict({"params_in_sync": False})
    assert report.ddp_verdict({"first_gradient_difference": 3, "first_parameter_difference": 3}) == "gradients differ after all_reduce"
    assert report.ddp_verdict({"first_gradient_difference": None, "first_parameter_difference": 7}) == "parameters differ, gradients equal"
    assert report.ddp_verdict({"first_gradient_difference": 9, "first_parameter_difference": 2}) == "parameters differ, gradients equal"
    assert report.ddp_verdict({"first_gradient_difference": None, "first_parameter_difference": None}) == "in sync"


def test_preflight_prefers_real_interfaces_and_falls_back_to_loopback(monkeypatch):
    import socket
    from types import SimpleNamespace as Address
    table = {"lo": [Address(family=socket.AF_INET, address="127.0.0.1")],
             "eth0": [Address(family=socket.AF_INET, address="10.1.2.3"), Address(family=socket.AF_INET6, address="fe80::1")],
             "dummy": [Address(family=socket.AF_INET, address="169.254.9.9")]}
    import psutil
    monkeypatch.setattr(psutil, "net_if_addrs", lambda: table)
    assert preflight.candidates(None) == [{"ifname": "eth0", "address": "10.1.2.3"}]
    assert preflight.candidates("lo") == [{"ifname": "lo", "address": "127.0.0.1"}]
    assert preflight.candidates("ib7") == []
    del table["eth0"]
    assert {c["ifname"] for c in preflight.candidates(None)} == {"lo", "dummy"}


def test_the_probes_child_reports_its_pci_address():
    from types import SimpleNamespace as Done
    seen = {}

    def fake(command, env, **_):
        seen["visible"] = env["CUDA_VISIBLE_DEVICES"]
        return Done(stdout="noise\npci=1b:00\n", stderr="", returncode=0)

    assert probe.child_pci("3", run=fake) == "1b:00" and seen["visible"] == "3"
    with pytest.raises(RuntimeError, match="no address.*exit code 1"):
        probe.child_pci("0", run=lambda *a, **k: Done(stdout="", stderr="boom", returncode=1))


# ---- the small diagnosis programs -----------------------------------------------------------------------
def test_the_supported_types_table_holds_for_gloo_in_this_torch(tmp_path):
    from gpubridge_b200.kit import gloo_dtypes
    found = gloo_dtypes.survey()
    assert gloo_dtypes.verdict(found) == []                        # every promised type sums and broadcasts exactly
    rows = found["rows"]
    assert all(rows[name] == {"all_reduce": "ok", "broadcast": "ok"} for name in ("float32", "bfloat16", "int64", "uint8"))
    # what the table leaves out is left out for a reason that still holds
    left_out = [name for name in gloo_dtypes.EXTRAS if name in rows and name != "bool"]
    assert any(rows[name]["all_reduce"] != "ok" for name in left_out)
    broken = dict(found, rows=dict(rows, float16={"all_reduce": "refused: x", "broadcast": "ok"}))
    assert gloo_dtypes.verdict(broken) == ["float16"]


def test_the_codec_diagnosis_finds_nothing_where_the_bits_match_and_explains_where_they_do_not(capsys):
    from gpubridge_b200 import compression as C
    from gpubridge_b200.kit import codec_diagnosis
    for mode, fmt in (("fp8", "ref"), ("fp8", "b200"), ("bf16", "ref")):
        assert codec_diagnosis.diagnose(mode, fmt, 5000, "cpu") == []
    assert codec_diagnosis.main(["--numel", "3000", "--device", "cpu"]) == 0
    assert "identical to the oracle" in capsys.readouterr().out

    def contracted(mode, x, residual, payload, fmt="ref"):
        """An implementation whose residual is rounded once (as a fused multiply-add would) and
        whose code of one value is off by one."""
        C.quantize_reference(mode, x, residual, payload, fmt)
        residual[100] = residual[100] + residual[100].abs() * 2.0 ** -22 + 1e-12
        head = 4 * C.n_blocks(x.numel(), fmt)
        payload[head + 200] ^= 1

    found = codec_diagnosis.diagnose("fp8", "ref", 5000, "cpu", quantize=contracted)
    text = "\n".join(found)
    assert len(found) == 2 and "value 100 (block 0)" in text and "value 200 (block 0)" in text
    assert "a fused multiply-add would leave" in text and "oracle 0x" in text and "residual" in text

    def other_scale(mode, x, residual, payload, fmt="ref"):
        C.quantize_reference(mode, x, residual, payload, fmt)
        payload[:4].view(torch.float32).mul_(2)

    assert any(line.startswith("block 0: scale") for line in codec_diagnosis.diagnose("fp8", "ref", 1000, "cpu", quantize=other_scale))
