"""Host cost per collective call of the two front ends of the torch backend.

    python -m gpubridge_b200.bench.bench_front_end                       # one GPU, a team of one
    torchrun --nproc-per-node 8 -m gpubridge_b200.bench.bench_front_end --backend gpubridge
    torchrun --nproc-per-node 8 -m gpubridge_b200.bench.bench_front_end --backend gpubridge_native

One process: the same fused kernels on a team of one, reached three ways - the Python fabric
call, the C++ backend with ``wait()``, and the C++ backend issued on the communication stream
itself (no event hand-over) - so the difference is the front end's.  Under torchrun:
``dist.all_reduce`` of a small tensor through the named backend.  Reported per case: host
microseconds per call while the GPU runs behind (what the launching thread pays), and
microseconds per call including the device (what a loop of dependent calls pays).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

import torch
import torch.distributed as dist


class _OnlyTheEngine:
    """What the C++ backend asks of its Python group, for a team of one."""

    def __init__(self, fabric) -> None:
        self.fabric = fabric

    def _native_team(self):
        f = self.fabric
        return (f.engine(), f.comm_stream.cuda_stream, f.device.index, f.overlap_blocks, [0])

    def _native_failed(self) -> None:
        self.fabric.check()

    def shutdown(self) -> None:
        pass


def measure(fn, device, calls: int) -> dict:
    for _ in range(200):
        fn()
    torch.cuda.synchronize(device)
    t0 = time.perf_counter()
    for _ in range(calls):
        fn()
    host = (time.perf_counter() - t0) / calls * 1e6
    torch.cuda.synchronize(device)
    total = (time.perf_counter() - t0) / calls * 1e6
    return {"host_us_per_call": round(host, 2), "with_device_us_per_call": round(total, 2)}


def one_process(args) -> dict:
    from gpubridge_b200.ops import _build_c10d, fabric as fabric_mod
    device = torch.device("cuda", 0)
    fabric = fabric_mod.create_single(device)
    backend = _build_c10d.load().GbBackend(0, 1, _OnlyTheEngine(fabric))
    t = torch.ones(args.numel, device=device)
    opts = dist.AllreduceOptions()
    out = {}
    try:
        out["python fabric.all_reduce"] = measure(lambda: fabric.all_reduce(t), device, args.calls)
        out["c++ backend.allreduce().wait()"] = measure(lambda: backend.allreduce([t], opts).wait(), device, args.calls)
        with torch.cuda.stream(fabric.comm_stream):
            out["c++ backend.allreduce() on the communication stream"] = measure(
                lambda: backend.allreduce([t], opts), device, args.calls)
        fabric.check()
    finally:
        backend.forget()
        torch.cuda.synchronize(device)
        fabric.close()
    return out


def under_torchrun(args) -> dict:
    if args.backend == "gpubridge_native":
        import gpubridge_b200.native_backend  # noqa: F401 - registers the name
    else:
        import gpubridge_b200  # noqa: F401
    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(device)
    dist.init_process_group(args.backend)
    t = torch.ones(args.numel, device=device)
    try:
        return {f"dist.all_reduce, backend={args.backend}, {dist.get_world_size()} ranks":
                measure(lambda: dist.all_reduce(t), device, args.calls)}
    finally:
        dist.destroy_process_group()


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--backend", default="gpubridge", choices=("gpubridge", "gpubridge_native", "nccl"))
    ap.add_argument("--calls", type=int, default=3000)
    ap.add_argument("--numel", type=int, default=256)
    ap.add_argument("--json")
    args = ap.parse_args(argv)
    if not torch.cuda.is_available():
        print("bench_front_end needs a GPU (the host cost of a launch is what it measures)")
        return 2
    result = under_torchrun(args) if "WORLD_SIZE" in os.environ else one_process(args)
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps(result, indent=1))
        if args.json:
            with open(args.json, "w") as fh:
                json.dump(result, fh, indent=1)
    return 0


if __name__ == "__main__":
    sys.exit(main())
