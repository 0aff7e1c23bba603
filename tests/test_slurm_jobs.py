"""The kit's Slurm jobs, end to end on a pretend cluster (tests/fake_slurm.py): CPU ranks, every
node on this machine.  What a cluster would run is what runs here - the same scripts, the
same programs - so a broken flag or path shows up before an allocation is spent on it."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SLURM = os.path.join(ROOT, "gpubridge_b200", "kit", "slurm")


@pytest.fixture
def cluster(tmp_path):
    tools = tmp_path / "bin"
    subprocess.run([sys.executable, os.path.join(ROOT, "tests", "fake_slurm.py"), "install", str(tools)], check=True)
    env = dict(os.environ, PATH=f"{tools}{os.pathsep}{os.environ['PATH']}", KIT_CPU="1", PYTHON=sys.executable,
               FAKE_SLURM_LOG=str(tmp_path / "slurm.log"), OMP_NUM_THREADS="1", KIT_TIMEOUT="120",
               STEP_TIMEOUT="500")
    for name in ("GPUBRIDGE_SPLIT_TEST", "GPUBRIDGE_ISLANDS", "GPUBRIDGE_VENDOR", "GPUBRIDGE_BRIDGE"):
        env.pop(name, None)
    return env


def steps(directory):
    return {row["step"]: row for row in map(json.loads, (directory / "steps.jsonl").read_text().splitlines())}


def test_one_node_job_runs_the_runbook(cluster, tmp_path):
    out = tmp_path / "results"
    done = subprocess.run([os.path.join(SLURM, "submit.sh"), "--gpus", "2", "--out", str(out), "one_node"],
                          env=dict(cluster, RUNBOOK_ONLY="probe check-one-island summary-one-island"),
                          cwd=tmp_path, capture_output=True, text=True, timeout=900)
    assert done.returncode == 0, done.stdout + done.stderr
    job, job_id = (out / "jobs.txt").read_text().split()
    assert job == "one_node" and job_id.isdigit()
    journal = steps(out / "one_node")
    log = (out / "one_node" / "runbook.log").read_text()
    assert journal["runbook"]["ok"], log[-3000:]
    inner = steps(out / "one_node" / "runbook")
    assert set(inner) == {"probe", "check-one-island", "summary-one-island"} and all(r["ok"] for r in inner.values())
    slurm_out = next((out / "one_node").glob("slurm-*.out")).read_text()
    assert "[step] runbook ... ok" in slurm_out and "no problems found" in slurm_out
    assert "sbatch --parsable --gres=gpu:2" in (tmp_path / "slurm.log").read_text()


def test_two_node_job_bridges_two_pretend_boxes(cluster, tmp_path):
    out = tmp_path / "results"
    done = subprocess.run([os.path.join(SLURM, "submit.sh"), "--gpus", "2", "--out", str(out), "two_nodes"],
                          env=dict(cluster, PREFLIGHT_SECONDS="0.3", SWEEP_LARGEST="256K", MASTER_PORT="29620"),
                          cwd=tmp_path, capture_output=True, text=True, timeout=1500)
    assert done.returncode == 0, done.stdout + done.stderr
    journal = steps(out / "two_nodes")
    failed = {name: (out / "two_nodes" / row["log"]).read_text()[-1500:] for name, row in journal.items() if not row["ok"]}
    assert not failed, failed
    assert list(journal) == ["preflight", "check-one-island", "summary-one-island", "check-gloo", "summary-gloo",
                             "check-multitcp", "summary-multitcp", "sweep"]
    bridged = json.loads((out / "two_nodes" / "check-multitcp" / "rank0.json").read_text())
    assert bridged["run"]["bridge"] == "multitcp" and bridged["run"]["split_test"] == "node"
    assert [i["ranks"] for i in bridged["run"]["islands"]] == [[0, 1], [2, 3]]
    whole = json.loads((out / "two_nodes" / "check-one-island" / "rank0.json").read_text())
    assert len(whole["run"]["islands"]) == 1
    assert json.loads((out / "two_nodes" / "sweep.json").read_text())


def test_a_failing_step_is_recorded_and_the_job_goes_on(cluster, tmp_path):
    script = tmp_path / "job.sh"
    script.write_text(f'OUT="{tmp_path}/o"\n. "{SLURM}/common.sh"\nstep good true\nstep bad bash -c "echo boom; exit 3"\n'
                      'STEP_TIMEOUT=1 step slow sleep 30\nstep after true\nfinish\n')
    done = subprocess.run(["bash", str(script)], env=cluster, capture_output=True, text=True, timeout=120)
    assert done.returncode == 1
    journal = steps(tmp_path / "o")
    assert [journal[s]["ok"] for s in ("good", "bad", "slow", "after")] == [True, False, False, True]
    assert journal["bad"]["exit_code"] == 3 and journal["slow"]["exit_code"] is None
    assert "step bad: FAILED (exit code 3" in done.stdout and "step slow: FAILED (ran past its limit" in done.stdout


def test_two_machines_without_a_scheduler(cluster, tmp_path):
    """node.sh on "both machines" at once (this one, twice): each side's host name is made up,
    so the two sides form two islands joined by the host bridge."""
    out = tmp_path / "pair"
    sides = []
    for node in (0, 1):
        env = dict(cluster, NODE_RANK=str(node), MASTER_ADDR="127.0.0.1", OUT=str(out), GPUS="2",
                   MASTER_PORT="29640", PREFLIGHT_SECONDS="0.3", SWEEP_LARGEST="256K",
                   GPUBRIDGE_SIM_HOSTNAME=f"machine-{node}")
        sides.append(subprocess.Popen([os.path.join(SLURM, "node.sh")], env=env, cwd=tmp_path,
                                      stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    texts = [side.communicate(timeout=1200)[0] for side in sides]
    assert [side.returncode for side in sides] == [0, 0], texts
    for node in (0, 1):
        journal = steps(out / f"node{node}")
        assert list(journal) == ["preflight", "check-gloo", "check-multitcp", "sweep"]
        assert all(row["ok"] for row in journal.values()), texts[node]
    record = json.loads((out / "check-multitcp" / "rank3.json").read_text())
    assert record["run"]["bridge"] == "multitcp"
    assert [i["ranks"] for i in record["run"]["islands"]] == [[0, 1], [2, 3]]
