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
           "--trials", "2", "--seconds", "1", "--phases", "--candidates", "sharded-bridge",
           "--json", str(out), "--write-thresholds", str(rules)]
    done = subprocess.run(cmd, env=env, cwd=ROOT, capture_output=True, text=True, timeout=300)
    assert done.returncode == 0, done.stderr[-3000:]
    rows = json.loads(out.read_text())
    assert {r["target"] for r in rows} >= {"ours", "compression:fp8", "policy:flat-gloo"}
    assert "policy:sharded-bridge" in {r["target"] for r in rows}            # from --candidates
    ours = [r for r in rows if r["target"] == "ours"]
    assert all({"island-reduce", "bridge", "island-broadcast", "total"} <= set(r["phases_ms"]) for r in ours)
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
                           "--profile", "4", "--out", str(out)], env=env, cwd=ROOT, capture_output=True, text=True,
                          timeout=300)
    assert done.returncode == 0, done.stderr[-3000:]
    record = json.loads(out.read_text())
    assert record["stub_comm"] and "reduce-bridge-broadcast/sync/plain" in record["us_per_call"]
    hot = record["profiles"]["reduce-bridge-broadcast/profile"]
    assert len(hot) == 4 and all(row["own_us_per_call"] > 0 for row in hot)
    assert any("all_reduce" in row["function"] for row in hot)


def test_import_time_bench(tmp_path):
    from gpubridge_b200.bench import bench_import
    out = tmp_path / "import.json"
    assert bench_import.main(["--runs", "1", "--out", str(out)]) == 0
    record = json.loads(out.read_text())
    assert record["with_package_s"] > 0 and record["slowest_modules"]
    assert all(row["module"].startswith("gpubridge_b200") for row in record["slowest_modules"])


def test_train_bench_shares():
    from gpubridge_b200.bench.train_bench import even_shares, speed_shares
    import pytest
    assert even_shares(7, 3) == [3, 2, 2]
    with pytest.raises(ValueError):
        even_shares(2, 3)
    assert speed_shares(12, [1.0, 2.0]) == [8, 4]          # twice as fast: twice the samples
    assert speed_shares(5, [1.0, 1.0]) == [3, 2]           # ties go to the lower rank
    assert speed_shares(6, [1.0, 100.0], floor=2) == [4, 2]
    shares = speed_shares(64, [0.8, 1.0, 1.3, 2.1])
    assert sum(shares) == 64 and shares == sorted(shares, reverse=True)
    worst = max(s * t for s, t in zip(shares, [0.8, 1.0, 1.3, 2.1]))
    assert all(worst <= (s + 1) * t + 1e-9 for s, t in zip(shares, [0.8, 1.0, 1.3, 2.1]))
    with pytest.raises(ValueError):
        speed_shares(3, [1.0, 0.0])


def test_accumulated_step_equals_one_step():
    """Micro-batches weighted by their share give the update of one backward over the whole batch."""
    import torch
    from gpubridge_b200.parallel.trainer import DataParallelTrainer

    def make():
        torch.manual_seed(3)
        return torch.nn.Sequential(torch.nn.Linear(6, 5), torch.nn.Tanh(), torch.nn.Linear(5, 1))

    x, y = torch.randn(8, 6), torch.randn(8, 1)
    mean = lambda m, a, b: torch.nn.functional.mse_loss(m(a), b)                      # noqa: E731
    share = lambda m, a, b: torch.nn.functional.mse_loss(m(a), b) * (a.shape[0] / 8)  # noqa: E731
    whole = DataParallelTrainer(make(), mean, autocast=None, exchange=False)
    parts = DataParallelTrainer(make(), share, autocast=None, exchange=False)
    for _ in range(3):
        a = whole.step(x, y)
        b = parts.step_accumulated([(x[:3], y[:3]), (x[3:4], y[3:4]), (x[4:], y[4:])])
        assert torch.allclose(a, b, atol=1e-6)
    assert torch.allclose(whole.flat_param, parts.flat_param, atol=1e-6)


def test_train_bench_two_ranks(tmp_path):
    env = dict(os.environ, PYTHONPATH=ROOT, OMP_NUM_THREADS="1", GPUBRIDGE_VENDOR="nvidia",
               GPUBRIDGE_SPLIT_TEST="half")
    for port, extra in ((29741, ["--model", "tiny-gpt", "--engine", "trainer", "--batch-sizes", "3,5",
                                 "--accumulate", "2"]),
                        (29742, ["--model", "tiny-resnet", "--global-batch", "7", "--controlled"]),
                        (29743, ["--model", "tiny-gpt", "--grad-sync", "native"])):
        out = tmp_path / f"tb{port}.json"
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
               "--master-addr", "127.0.0.1", "--master-port", str(port), "-m",
               "gpubridge_b200.bench.train_bench", *extra, "--steps", "3", "--warmup-steps", "1",
               "--comm-trials", "2", "--json", str(out)]
        done = subprocess.run(cmd, env=env, cwd=ROOT, capture_output=True, text=True, timeout=300)
        assert done.returncode == 0, done.stderr[-3000:]
        r = json.loads(out.read_text())
        assert r["params_identical"] and r["params_finite"] and r["params_sum_spread"] == 0.0
        assert r["exchanges_per_step"] == len(r["bucket_bytes"]) >= 1
        assert r["samples_per_s"] > 0 and len(r["ranks"]) == 2
        assert abs(r["ddp_step_ms"] - r["slowest_compute_ms"] - r["exposed_comm_ms"]) < 2e-3
        if "--batch-sizes" in extra:
            assert [x["batch"] for x in r["ranks"]] == [3, 5] and r["ranks"][1]["micro_batches"] == [3, 2]
        if "--controlled" in extra:
            assert r["controlled"]["initial_parameters"] and r["dtype"] == "fp32" and r["split"] == "even"
        if "native" in extra:
            assert "stand-in" in r["note"]


def test_recorded_train_dp_and_report(tmp_path):
    """Same data at any scale: a single process, DDP with unequal shares and HSDP land on the
    same loss curve, and the report lays them side by side."""
    from gpubridge_b200.bench.train_dp import shares_for
    from gpubridge_b200.kit import report
    assert shares_for([1, 1, 1], 8) == [3, 3, 2] and shares_for([3.0, 1.0], 8) == [6, 2]
    assert sum(shares_for([0.7, 1.9, 1.1], 17)) == 17 and min(shares_for([100.0, 1.0], 5)) == 1
    env = dict(os.environ, PYTHONPATH=ROOT, OMP_NUM_THREADS="1", GPUBRIDGE_VENDOR="nvidia",
               GPUBRIDGE_SPLIT_TEST="half")
    runs = tmp_path / "runs"
    runs.mkdir()
    for port, ranks, mode, extra in ((29751, 1, "single", ["--micro", "3"]),
                                     (29752, 2, "ddp", ["--shares", "5,3"]),
                                     (29754, 4, "hsdp", []),
                                     (29755, 2, "fused", [])):
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={ranks}",
               "--master-addr", "127.0.0.1", "--master-port", str(port), "-m", "gpubridge_b200.bench.train_dp",
               "--model", "llama-tiny", "--mode", mode, "--seq", "16", "--steps", "6", "--warmup", "1",
               "--global-batch", "8", "--check-every", "3", "--lr", "3e-3", *extra,
               "--json", str(runs / f"dp_{mode}.json")]
        done = subprocess.run(cmd, env=env, cwd=ROOT, capture_output=True, text=True, timeout=400)
        assert done.returncode == 0, done.stderr[-3000:]
    got = {m: json.loads((runs / f"dp_{m}.json").read_text()) for m in ("single", "ddp", "hsdp", "fused")}
    assert got["fused"]["sharded_layers"] == 14 and got["fused"]["parameters_identical"] is True
    assert got["ddp"]["shares"] == [5, 3] and got["ddp"]["parameters_identical"] is True
    assert got["hsdp"]["parameters_identical"] is True and len(got["hsdp"]["parameter_checks"]) == 2
    for mode in ("ddp", "hsdp", "fused"):
        gaps = [abs(a - b) for a, b in zip(got[mode]["losses"], got["single"]["losses"])]
        assert max(gaps) < 1e-4, (mode, gaps)
    assert got["single"]["losses"][-1] < got["single"]["losses"][0]
    assert report.main(["dp", str(runs), "--out", str(tmp_path / "rep"), "--tail", "3"]) == 0
    text = (tmp_path / "rep" / "dp_report.md").read_text()
    assert "(baseline)" in text and "[5, 3]" in text and "| yes |" in text
    assert (tmp_path / "rep" / "loss_curves.csv").read_text().count("\n") == 8
    assert (tmp_path / "rep" / "loss_curves.svg").read_text().count("<polyline") == 4


def test_ddp_divergence_report(tmp_path, capsys):
    from gpubridge_b200.kit import report
    base = {"world_size": 2, "engine": "ddp", "samples_per_sec": 10.0, "params_in_sync": True,
            "first_gradient_difference": None, "first_parameter_difference": None}
    rows = {"a": base, "b": {**base, "params_in_sync": False, "first_gradient_difference": 3,
                             "first_parameter_difference": 3},
            "c": {**base, "params_in_sync": False, "first_parameter_difference": 7},
            "old": {"world_size": 2, "samples_per_sec": 1.0, "params_in_sync": True}}
    for name, row in rows.items():
        (tmp_path / f"{name}.json").write_text(json.dumps(row))
    assert report.main(["ddp", str(tmp_path), "--out", str(tmp_path / "o")]) == 1
    text = capsys.readouterr().out
    assert "| a | 2 | ddp | - | 10.0 | - | - | in sync |" in text
    assert "step 3 | step 3 | gradients differ after all_reduce" in text
    assert "| - | step 7 | parameters differ, gradients equal" in text
    assert "no per-step check" in text and "2 of 4 runs in sync" in text
    assert (tmp_path / "o" / "train_ddp_report.md").exists()
