"""Pipeline parallelism through backend="gpubridge" on CPU ranks: the losses equal those of
the same pipeline on a plain Gloo group bit for bit (GPipe and 1F1B), and the balanced split
runs end to end."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(port, *args, nproc=2):
    env = dict(os.environ, PYTHONPATH=ROOT, OMP_NUM_THREADS="1", GPUBRIDGE_VENDOR="nvidia",
               GPUBRIDGE_SPLIT_TEST="half")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1",
           f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1", "--master-port", str(port),
           "-m", "gpubridge_b200.bench.train_pipeline", "--model", "llama-tiny", "--steps", "3",
           *args]
    done = subprocess.run(cmd, env=env, cwd=ROOT, capture_output=True, text=True, timeout=300)
    assert done.returncode == 0, done.stderr[-3000:]
    line = [l for l in done.stdout.splitlines() if l.startswith('{"bench"')][-1]
    return json.loads(line)


@pytest.mark.parametrize("schedule", ["gpipe", "1f1b"])
def test_losses_match_gloo(schedule):
    ours = _run(29791, "--schedule", schedule)
    gloo = _run(29792, "--schedule", schedule, "--backend", "gloo")
    assert ours["losses"] == gloo["losses"]
    assert ours["split"] == [1, 1] and len(ours["losses"]) == 3


def test_auto_split(tmp_path):
    out = tmp_path / "pp.json"
    record = _run(29793, "--split", "auto", "--json", str(out))
    saved = json.loads(out.read_text())
    assert sum(record["split"]) == 2 and saved["profile"]["predicted_bottleneck_ms"] > 0
    assert len(saved["profile"]["link_bytes_per_ms"]) == 1


def test_hand_scheduled_1f1b_over_batched_p2p(tmp_path):
    """The Megatron-style schedule: four stages, fewer / as many / more micro-batches than
    stages, every step's loss against one process; once through the C++ front end."""
    import json
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, PYTHONPATH=root, OMP_NUM_THREADS="1", GPUBRIDGE_VENDOR="nvidia",
               GPUBRIDGE_SPLIT_TEST="half")
    for port, micro, backend in ((29661, 2, "gpubridge"), (29662, 4, "gpubridge_native"), (29663, 8, "gpubridge")):
        out = tmp_path / f"pp{micro}.json"
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=4",
               "--master-addr", "127.0.0.1", "--master-port", str(port), "-m",
               "gpubridge_b200.bench.train_pp_p2p", "--model", "llama-mini", "--verify", "--steps", "3",
               "--warmup-steps", "1", "--seq", "16", "--microbatches", str(micro), "--backend", backend,
               "--json", str(out)]
        done = subprocess.run(cmd, env=env, cwd=root, capture_output=True, text=True, timeout=400)
        assert done.returncode == 0, done.stderr[-3000:]
        record = json.loads(out.read_text())
        assert record["stages"] == 4 and record["largest_loss_gap_to_one_process"] < 1e-4
        assert record["losses"][-1] < record["losses"][0]
        # warm-up receives + steady-state pairs + cool-down: first stage has the fewest batches
        assert record["p2p_batches_per_step"] >= micro
