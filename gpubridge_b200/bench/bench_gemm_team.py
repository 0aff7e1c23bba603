"""The two fused GEMM kernels on a team against what they replace, shape by shape.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 4 --master-addr 127.0.0.1 \
        -m gpubridge_b200.bench.bench_gemm_team [--shapes 8192x5632x2048,...] [--trials 10]

Per shape ``M x N x K`` (the forward of a row-sharded Linear: ``x`` is ``[M, K]``, every rank
holds ``N / world`` rows of the ``[N, K]`` weight):

* ``allgather_gemm``: the fused kernel (communication CTAs pull the peers' shards while the
  tensor cores work on the shards that are there) against NCCL ``all_gather_into_tensor``
  followed by cuBLAS ``F.linear``, and against this library's all-gather followed by cuBLAS;
* ``gemm_reduce_scatter``: the weight gradient ``dW = dY^T X`` (``[N, M] x [K, M]^T``) averaged
  and scattered by rows - one kernel - against cuBLAS ``matmul`` followed by NCCL
  ``reduce_scatter_tensor`` with AVG.

Each figure is the median over ``--trials`` of the slowest rank's device time (CUDA events on
the launching stream, barrier and synchronise before every trial, three warm-ups).  The
roofline of a fused kernel is the slower of its FLOPs at the measured cuBLAS rate and its
bytes over NVLink at the measured 770 GB/s per direction; both are printed.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import warnings

import torch
import torch.distributed as dist

SHAPES = "8192x5632x2048,8192x2048x5632,8192x8192x8192"
LINK_GBS = 770.0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--shapes", default=SHAPES)
    ap.add_argument("--trials", type=int, default=10)
    args = ap.parse_args(argv)
    import gpubridge_b200 as gb
    from gpubridge_b200.ops.gemm import AllGatherLinear, GemmReduceScatter
    local = int(os.environ.get("LOCAL_RANK", "0"))
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    with warnings.catch_warnings():
        warnings.simplefilter("ignore", gb.SplitTestWarning)
        topology = gb.init()
    fabric, world, rank = topology.fabric, topology.world_size, topology.rank
    nccl = topology.p2p_group
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    peak = 1600.0
    if os.path.exists(os.path.join(root, "MEASURED_PEAKS.json")):
        with open(os.path.join(root, "MEASURED_PEAKS.json")) as fh:
            peak = float(json.load(fh).get("bf16_tflops", peak))

    def slowest_us(fn) -> float:
        for _ in range(3):
            fn()
        samples = []
        for _ in range(args.trials):
            torch.cuda.synchronize(device)
            topology.world_group.barrier()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            fn()
            end.record()
            end.synchronize()
            t = torch.tensor([start.elapsed_time(end) * 1e3], dtype=torch.float64)
            topology.world_group.all_reduce(t, "max")
            samples.append(float(t))
        return round(statistics.median(samples), 1)

    for shape in args.shapes.split(","):
        M, N, K = (int(v) for v in shape.lower().split("x"))
        if N % world or fabric is None:
            continue
        torch.manual_seed(1 + rank)
        x = (torch.randn(M, K, device=device) * 0.05).to(torch.bfloat16)
        shard = (torch.randn(N // world, K, device=device) * 0.05).to(torch.bfloat16)
        whole = torch.empty(N, K, dtype=torch.bfloat16, device=device)
        row = {"M": M, "N": N, "K": K, "world": world}
        flops = 2.0 * M * N * K
        # ---- all-gather + GEMM
        try:
            fused = AllGatherLinear(fabric, N, K)
            row["allgather_gemm_fused_us"] = slowest_us(lambda: fused(x, shard))
            fused.check()
        except (ValueError, RuntimeError) as failure:
            row["allgather_gemm_fused_us"] = str(failure)[:120]

        def ours_then_cublas():
            gb.all_gather_into_tensor(whole.view(-1), shard.view(-1))
            return torch.nn.functional.linear(x, whole)

        row["our_allgather_then_cublas_us"] = slowest_us(ours_then_cublas)
        if nccl is not None:
            def nccl_then_cublas():
                nccl.all_gather_into(whole.view(-1), shard.view(-1))
                return torch.nn.functional.linear(x, whole)
            row["nccl_allgather_then_cublas_us"] = slowest_us(nccl_then_cublas)
        link_us = (N - N // world) * K * 2 / (LINK_GBS * 1e3)
        row["allgather_gemm_roofline_us"] = round(max(flops / (peak * 1e6), link_us), 1)
        # ---- GEMM + reduce-scatter: dW[N, K] = dY^T[N, M] @ X[M, K], rows scattered
        dy_t = (torch.randn(N, M, device=device) * 0.05).to(torch.bfloat16)
        x_t = x.t().contiguous()                                   # [K, M]: contraction-major
        both = GemmReduceScatter(fabric)
        if both.fits(N, K, M):
            row["gemm_reduce_scatter_fused_us"] = slowest_us(lambda: both(dy_t, x_t, divide=world))
            both.check()
        else:
            row["gemm_reduce_scatter_fused_us"] = "does not fit the staging region"
        if nccl is not None:
            out = torch.empty(N // world, K, dtype=torch.bfloat16, device=device)

            def cublas_then_nccl():
                full = dy_t @ x_t.t()
                nccl.reduce_scatter_into(out.view(-1), full.view(-1), dist.ReduceOp.AVG)
            try:
                row["cublas_then_nccl_reduce_scatter_us"] = slowest_us(cublas_then_nccl)
            except Exception as failure:  # noqa: BLE001
                row["cublas_then_nccl_reduce_scatter_us"] = str(failure)[:120]
        link_us = (N - N // world) * K * 2 / (LINK_GBS * 1e3)
        row["gemm_reduce_scatter_roofline_us"] = round(max(flops / (peak * 1e6), link_us), 1)
        if rank == 0:
            print(json.dumps(row), flush=True)
    gb.destroy()
    return 0


if __name__ == "__main__":
    sys.exit(main())
