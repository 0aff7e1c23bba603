"""All-reduce across simulated islands on CPU: no GPU, no torchrun.

Each spawned process names its vendor through GPUBRIDGE_VENDOR, so discovery, leader
election and the bridged all-reduce run exactly as on a mixed machine, with Gloo standing in
for the island library.  Pass the vendors on the command line to try other shapes:

    python examples/simulate_islands.py                       # nvidia nvidia amd amd
    python examples/simulate_islands.py nvidia amd amd amd nvidia
    GPUBRIDGE_BRIDGE_COMPRESSION=fp8 python examples/simulate_islands.py
    python examples/simulate_islands.py --bridge multitcp     # the native TCP worker between the leaders
"""
from __future__ import annotations

import os
import sys
import tempfile

import torch
import torch.multiprocessing as mp

import os as _os, sys as _sys
_sys.path.insert(0, _os.path.dirname(_os.path.dirname(_os.path.abspath(__file__))))  # run from a checkout
import gpubridge_b200 as gb


def worker(rank: int, vendors: list[str], rendezvous: str, bridge: str | None) -> None:
    os.environ["GPUBRIDGE_VENDOR"] = vendors[rank]
    topo = gb.init(init_method=f"file://{rendezvous}", rank=rank, world_size=len(vendors), bridge=bridge)
    if rank == 0:
        for island in topo.layout.islands:
            print(f"island {island.vendor:<8} ranks {list(island.ranks)}  leader {island.leader}")
        print(f"bridge link between leaders {list(topo.layout.bridge_ranks)} over {topo.peers[0].bridge}, "
              f"policy {topo.policy_name}\n", flush=True)
    gb.barrier()
    t = torch.full((4,), float(rank + 1))
    gb.all_reduce(t)
    for turn in range(topo.world_size):            # print in rank order
        if turn == rank:
            print(f"rank {rank} ({topo.vendor}, {'leader' if topo.is_leader else 'member'}): "
                  f"{t.tolist()}", flush=True)
        gb.barrier()
    want = float(sum(range(1, topo.world_size + 1)))
    verdict = torch.tensor([float(bool((t == want).all()))])
    gb.all_reduce(verdict, gb.ReduceOp.MIN)
    if rank == 0:
        print(f"\nexpected {want} everywhere: {'all ranks match' if verdict.item() else 'MISMATCH'}")
    gb.destroy()
    if not verdict.item():
        sys.exit(1)


if __name__ == "__main__":
    words = sys.argv[1:]
    bridge = None
    if "--bridge" in words:
        at = words.index("--bridge")
        bridge = words[at + 1]
        del words[at:at + 2]
    vendors = words or ["nvidia", "nvidia", "amd", "amd"]
    with tempfile.TemporaryDirectory() as tmp:
        mp.spawn(worker, args=(vendors, os.path.join(tmp, "rendezvous"), bridge), nprocs=len(vendors))
