"""The benchmark programs on CPU ranks: the sweep (targets, compression check, thresholds
file), the matrix merger and the per-call cost table run end to end."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_sweep_matrix_and_thresholds(tmp_path):
    env = dict(os.environ, PYTHONPATH=ROOT, OMP_NUM_THREADS="1", GPUBRIDGE_VENDOR="nvidia",
               GPUBRIDGE_SPLIT_TEST="half")
    out, rules = tmp_path / "sweep.json", tmp_path / "thresholds.json"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=4",
           "--master-addr", "127.0.0.1", "--master-port", "29727", "-m",
           "gpubridge_b200.bench.bench_all_reduce", "--smallest", "4K", "--largest", "64K",
           "--targets", "ours,compression:fp8,policy:flat-gloo,policy:reduce-bridge-broadcast",
           "--trials", "2", "--seconds", "1", "--json", str(out), "--write-thresholds", str(rules)]
    done = subprocess.run(cmd, env=env, cwd=ROOT, capture_output=True, text=True, timeout=300)
    assert done.returncode == 0, done.stderr[-3000:]
    rows = json.loads(out.read_text())
    assert {r["target"] for r in rows} >= {"ours", "compression:fp8", "policy:flat-gloo"}
    coded = [r for r in rows if r["target"] == "compression:fp8"]
    assert all(r["identical_bits"] and 0 < r["max_rel_error"] < 0.2 for r in coded)
    saved = json.loads(rules.read_text())
    assert saved["gpubridge_thresholds"] == 1 and saved["rules"][-1]["max_bytes"] is None
    from gpubridge_b200.bench import bench_matrix
    assert bench_matrix.main([f"cpu={out}", "--baseline", "cpu/policy:flat-gloo",
                              "--out", str(tmp_path / "matrix")]) == 0
    matrix = json.loads((tmp_path / "matrix" / "matrix.json").read_text())
    assert matrix["baseline"] == "cpu/policy:flat-gloo" and matrix["rows"]
    assert "under 256 KB" in (tmp_path / "matrix" / "matrix.md").read_text()


def test_per_call_table(tmp_path):
    env = dict(os.environ, PYTHONPATH=ROOT)
    for name in ("GPUBRIDGE_SPLIT_TEST", "GPUBRIDGE_ISLANDS", "GPUBRIDGE_VENDOR"):
        env.pop(name, None)
    out = tmp_path / "per_call.json"
    done = subprocess.run([sys.executable, "-m", "gpubridge_b200.bench.bench_per_call", "--calls", "20",
                           "--rounds", "1", "--stub-comm", "--policies", "reduce-bridge-broadcast",
                           "--out", str(out)], env=env, cwd=ROOT, capture_output=True, text=True,
                          timeout=300)
    assert done.returncode == 0, done.stderr[-3000:]
    record = json.loads(out.read_text())
    assert record["stub_comm"] and "reduce-bridge-broadcast/sync/plain" in record["us_per_call"]
