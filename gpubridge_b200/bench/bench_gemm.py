"""The tcgen05 all-gather GEMM on one GPU against cuBLAS, shape by shape.

    python -m gpubridge_b200.bench.bench_gemm [--shapes 8192x8192x8192,8192x5632x2048] [--trials 10]

A team of one runs the same kernels without peers, so this times the GEMM itself: the CTA-pair
kernel (``cta_group::2``), the single-CTA kernel and ``torch.matmul`` (cuBLAS) on the same
operands, each as the median of ``--trials`` launches between CUDA events after three
warm-ups, with a buffer larger than L2 written between launches so no launch starts on
operands the previous one left in cache.  Rows give TFLOP/s, the fraction of cuBLAS on this
GPU and - when ``MEASURED_PEAKS.json`` sits at the repository root - of the measured bf16 peak.
``GPUBRIDGE_GEMM_GROUP`` (n-tiles per band of the tile walk; 0 = n outer, m inner) and
``GPUBRIDGE_GEMM_PROBE=1`` (load operands, issue no MMA: the ingest rate alone) are read by
the library at its first launch: set them per process.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys

import torch

SHAPES = "8192x8192x8192,8192x5632x2048,8192x2048x5632,4096x14336x4096"


def median_us(fn, trials: int, flush: torch.Tensor) -> float:
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    samples = []
    for _ in range(trials):
        flush.add_(1.0)                              # evicts the operands from L2
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        fn()
        end.record()
        end.synchronize()
        samples.append(start.elapsed_time(end) * 1e3)
    return statistics.median(samples)


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    parser.add_argument("--shapes", default=SHAPES, help="MxNxK, comma separated")
    parser.add_argument("--trials", type=int, default=10)
    parser.add_argument("--kernels", default="pair,one,cublas")
    args = parser.parse_args(argv)
    from gpubridge_b200.ops import fabric as fabric_mod
    from gpubridge_b200.ops.gemm import AllGatherLinear
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    peak = None
    if os.path.exists(os.path.join(root, "MEASURED_PEAKS.json")):
        with open(os.path.join(root, "MEASURED_PEAKS.json")) as fh:
            peak = json.load(fh).get("bf16_tflops")
    team = fabric_mod.create_single(device)
    flush = torch.zeros(64 << 20, device=device)                   # 256 MiB
    try:
        for shape in args.shapes.split(","):
            M, N, K = (int(v) for v in shape.lower().split("x"))
            x = (torch.randn(M, K, device=device) * 0.5).to(torch.bfloat16)
            w = (torch.randn(N, K, device=device) * 0.5).to(torch.bfloat16)
            flops = 2.0 * M * N * K
            row = {"M": M, "N": N, "K": K, "group": os.environ.get("GPUBRIDGE_GEMM_GROUP", "default"),
                   "probe": os.environ.get("GPUBRIDGE_GEMM_PROBE", "0")}
            results = {}
            for kernel in args.kernels.split(","):
                if kernel == "cublas":
                    fn = lambda: torch.matmul(x, w.t())                         # noqa: E731
                else:
                    op = AllGatherLinear(team, N, K, pair=kernel == "pair")
                    fn = lambda op=op: op(x, w)                                 # noqa: E731
                us = median_us(fn, args.trials, flush)
                results[kernel] = fn()
                row[kernel] = {"us": round(us, 1), "tflops": round(flops / us / 1e6, 1)}
                if kernel != "cublas":
                    op.check()
            if "cublas" in row:
                for kernel in ("pair", "one"):
                    if kernel in row:
                        row[kernel]["of_cublas"] = round(row[kernel]["tflops"] / row["cublas"]["tflops"], 3)
                        if row["probe"] == "0":
                            worst = (results[kernel].float() - results["cublas"].float()).abs().max()
                            row[kernel]["max_abs_diff_to_cublas"] = round(float(worst), 4)
            if peak:
                for kernel in ("pair", "one", "cublas"):
                    if kernel in row:
                        row[kernel]["of_measured_peak"] = round(row[kernel]["tflops"] / peak, 3)
            print(json.dumps(row), flush=True)
    finally:
        torch.cuda.synchronize()
        team.check()
        team.close()
    return 0


if __name__ == "__main__":
    sys.exit(main())
