"""Link probe: NVLink store / load bandwidth from inside a kernel, local copy bandwidth and
the cost of one team barrier, per grid size.  The numbers size the role split of the
pipelined collectives and the device-side timeouts (the reference has a TCP bandwidth / RTT
probe for its host bridge: scripts/gpu/preflight.py).

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 \
        -m gpubridge_b200.bench.bench_link [grids, e.g. 1,8,32,128]

``ring-`` rows move the same bytes through the bulk-copy ring (TMA loads into shared memory,
ordinary stores out of it) instead of loads into registers.
"""
from __future__ import annotations

import json
import sys
import warnings

import torch

import gpubridge_b200 as gb


def main() -> int:
    with warnings.catch_warnings():
        warnings.simplefilter("ignore", gb.SplitTestWarning)
        topology = gb.init()
    fabric = topology.fabric
    rows = []
    try:
        if fabric is None:
            raise SystemExit("bench_link needs a GPU team with a fabric")
        nbytes = min(fabric.len_ha, fabric.len_hb, fabric.len_hc, 64 << 20)

        def timed(kind: str, grid: int, n: int, repeat: int) -> float:
            with torch.cuda.stream(fabric.comm_stream):
                for _ in range(2):
                    fabric.probe(kind, n, grid, repeat)
                start, end = (torch.cuda.Event(enable_timing=True) for _ in range(2))
                start.record()
                fabric.probe(kind, n, grid, repeat)
                end.record()
                end.synchronize()
            t = torch.tensor([start.elapsed_time(end)], dtype=torch.float64)
            topology.world_group.all_reduce(t, "max")
            return float(t)

        grids = [int(g) for g in (sys.argv[1] if len(sys.argv) > 1 else "1,4,8,16,32,64,128").split(",")]
        for grid in grids:
            base = timed("barrier", grid, 0, 1)                    # launch + two barriers
            ms = timed("barrier", grid, 200, 1)
            rows.append({"probe": "barrier", "grid": grid,
                         "us_per_barrier": round((ms - base) * 1000 / 200, 2),
                         "launch_plus_2_barriers_us": round(base * 1000, 1)})
            for kind in ("store", "ring-store", "load", "ring-load", "copy", "ring-copy", "mixed",
                         "mixed3"):
                if kind.startswith("mixed") and grid < 8:
                    continue
                repeat = 8
                ms = timed(kind, grid, nbytes, repeat) - base
                # mixed: every group moves nbytes * repeat; the rate is per group
                rows.append({"probe": kind, "grid": grid, "bytes": nbytes,
                             "gbs": round(nbytes * repeat / (ms * 1e-3) / 1e9, 1)})
        fabric.check()
    finally:
        gb.destroy()
    if topology.rank == 0:
        for row in rows:
            print(json.dumps(row), flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
