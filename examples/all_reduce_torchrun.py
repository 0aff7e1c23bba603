"""The smallest program: one all-reduce, launched with torchrun on any number of GPUs.

    torchrun --nproc-per-node 8 examples/all_reduce_torchrun.py
    GPUBRIDGE_ISLANDS=4,4 torchrun --nproc-per-node 8 examples/all_reduce_torchrun.py

With GPUs on one NVSwitch box the call is one fused kernel.  Without GPUs, name a vendor
(``GPUBRIDGE_VENDOR=nvidia``, optionally ``GPUBRIDGE_SPLIT_TEST=half``) to run on CPU.
"""
import torch

import os as _os, sys as _sys
_sys.path.insert(0, _os.path.dirname(_os.path.dirname(_os.path.abspath(__file__))))  # run from a checkout
import gpubridge_b200 as gb


def main() -> None:
    topo = gb.init()                                   # env:// rendezvous from torchrun
    t = torch.full((4,), float(topo.rank), device=topo.device)
    gb.all_reduce(t)
    role = "leader" if topo.is_leader else "member"
    path = "fused kernel" if topo.fabric is not None else "composed"
    print(f"rank {topo.rank} ({topo.vendor}, {role}, {path}): {t.tolist()}", flush=True)
    gb.destroy()


if __name__ == "__main__":
    main()
