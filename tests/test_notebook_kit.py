"""The notebook runner of the validation kit: its plan, a whole run with stand-in children
(features decide what is skipped, a failing step does not stop the rest, a step past its limit
is killed with its process group), the journal, the archive and the generated notebook."""
import json
import subprocess
import sys
import tarfile
import time
from pathlib import Path

from gpubridge_b200.kit import notebook as kit

ROOT = Path(__file__).resolve().parents[1]


def test_dry_run_lists_every_step_in_order():
    done = subprocess.run([sys.executable, str(ROOT / "gpubridge_b200" / "kit" / "notebook.py"), "--dry-run"],
                          capture_output=True, text=True, cwd="/")        # by path: it runs on its own
    assert done.returncode == 0, done.stderr
    names = [line[1:line.index("]")] for line in done.stdout.splitlines() if line.startswith("[")]
    assert names == list(kit.STEPS)
    assert "pytest tests -m gpu" in done.stdout and "kit.runbook" in done.stdout


def test_unknown_steps_are_refused(capsys):
    try:
        kit.main(["--only", "nonsense", "--dry-run"])
    except SystemExit as stop:
        assert stop.code == 2
    assert "unknown steps" in capsys.readouterr().err


def _runner(tmp_path, answers, **kwargs):
    calls = []

    def fake(cmd, limit, log, env=None):
        text = " ".join(cmd)
        calls.append(text)
        for needle, code in answers.items():
            if needle in text:
                return code
        return 0

    out = tmp_path / "results"
    out.mkdir()
    return kit.Runner(tmp_path, out, "/nowhere", "v0", run=fake, **kwargs), calls, out


def test_a_run_with_stand_in_children(tmp_path):
    # one GPU only; the test suite fails; the runbook runs past its limit
    answers = {"device_count() >= 2": 1, "can_device_access_peer": 1, "pytest tests -m gpu": 3,
               "kit.runbook": None}
    runner, calls, out = _runner(tmp_path, answers)
    rows = {name: runner.step(name) for name in kit.STEPS}
    assert rows["features"]["ok"] and runner.features["sm_100"] and not runner.features["two_gpus"]
    assert rows["gpu_tests"]["verdict"] == "failed" and "exit code 3" in rows["gpu_tests"]["note"]
    assert rows["runbook"]["verdict"] == "timeout"
    assert rows["fsdp2"]["verdict"] == "skipped" and "two_gpus" in rows["fsdp2"]["note"]
    assert rows["codec"]["verdict"] == "ok" and rows["tables"]["verdict"] == "ok"
    assert not any("fsdp2_torch_backend" in c for c in calls)          # skipped means not started
    journal = [json.loads(line) for line in (out / "steps.jsonl").read_text().splitlines()]
    assert [r["step"] for r in journal] == list(kit.STEPS)
    assert json.loads((out / "features.json").read_text())["two_gpus"] is False
    archive = Path(rows["package"]["note"])
    with tarfile.open(archive) as tar:
        assert "results/steps.jsonl" in tar.getnames()


def test_a_child_past_its_limit_is_killed_with_its_group(tmp_path):
    out = tmp_path / "results"
    out.mkdir()
    runner = kit.Runner(tmp_path, out, "/nowhere", "")
    marker = tmp_path / "grandchild-finished"
    late = tmp_path / "late.py"
    late.write_text(f"import time\ntime.sleep(3)\nopen({str(marker)!r}, 'w').write('x')\n")
    slow = tmp_path / "slow.py"
    slow.write_text(f"import subprocess, sys, time\nsubprocess.Popen([sys.executable, {str(late)!r}])\ntime.sleep(30)\n")
    started = time.monotonic()
    code = runner._child([sys.executable, str(slow)], 1.0, out / "slow.log")
    assert code is None and time.monotonic() - started < 10
    time.sleep(3.5)
    assert not marker.exists()                                         # the grandchild died too


def test_fetch_copies_a_local_checkout_without_its_history(tmp_path):
    source = tmp_path / "checkout"
    (source / ".git").mkdir(parents=True)
    (source / "pkg").mkdir()
    (source / "pkg" / "a.py").write_text("x = 1\n")
    out = tmp_path / "work" / "results"
    out.mkdir(parents=True)
    runner = kit.Runner(tmp_path / "work", out, str(source), "")
    assert runner.step("fetch")["verdict"] == "ok"
    assert (runner.src / "pkg" / "a.py").exists() and not (runner.src / ".git").exists()
    clone = kit.Runner(tmp_path / "w2", out, "https://example.org/x.git", "v9").commands("fetch")[0]
    assert clone[:2] == ["git", "clone"] and "v9" in clone


def test_the_generated_notebook_holds_this_file_and_a_cell_per_step(tmp_path):
    path = tmp_path / "kit.ipynb"
    assert kit.main(["--write-notebook", str(path), "--source", "https://example.org/x.git", "--ref", "v1"]) == 0
    book = json.loads(path.read_text())
    assert book["nbformat"] == 4
    code = ["".join(c["source"]) for c in book["cells"] if c["cell_type"] == "code"]
    assert code[0].startswith("%%writefile notebook_kit.py") and "class Runner" in code[0]
    assert len(code) == 1 + len(kit.STEPS)
    assert code[1].endswith("--only fetch") and "--ref v1" in code[1]
