"""Run one of the library's kernels a few times on one GPU, for ``ncu`` to capture.

    python -m gpubridge_b200.bench.profile_kernels hier|oneshot|switch|allgather|reducescatter|broadcast|xent|adamw|layernorm|quantize|dequantize|gemm

Sizes are small enough for a full-set capture to finish in about a minute but larger than
the 126 MB L2, so DRAM figures mean something.  ``hier`` and ``oneshot`` run one rank's side
of the fused all-reduce on a team of one (every "peer" access is local).
"""
from __future__ import annotations

import sys

import torch


def main(which: str) -> int:
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    if which in ("hier", "oneshot", "gemm", "switch", "allgather", "reducescatter", "broadcast"):
        from gpubridge_b200.ops import fabric as F
        team = F.create_single(device)
        if which == "gemm":
            from gpubridge_b200.ops.gemm import AllGatherLinear
            x = torch.randn(8192, 2048, device=device).to(torch.bfloat16)
            w = torch.randn(5632, 2048, device=device).to(torch.bfloat16)
            op = AllGatherLinear(team, 5632, 2048)
            for _ in range(4):
                op(x, w)
            torch.cuda.synchronize()
            op.check()
        elif which == "switch":
            # one rank's side of the in-switch all-reduce: a multicast object of one GPU
            if not team.enable_switch():
                team.close()
                raise SystemExit(f"switch: no multicast memory here ({team.switch_error})")
            t = torch.randn(48 << 20, device=device)              # 192 MiB: larger than L2
            for _ in range(4):
                team.all_reduce(t)
            torch.cuda.synchronize()
        elif which in ("allgather", "reducescatter", "broadcast"):
            # one rank's side of the copy-shaped collectives (stage, barrier, pull): 192 MiB
            t = torch.randn(48 << 20, device=device)
            out = torch.empty_like(t)
            for _ in range(4):
                if which == "allgather":
                    team.all_gather(out, t)
                elif which == "reducescatter":
                    team.reduce_scatter(out, t)
                else:
                    team.broadcast(t, 0)
            torch.cuda.synchronize()
        else:
            n = (32 << 20) if which == "hier" else (64 << 10)
            t = torch.randn(n, device=device)
            for _ in range(4):
                team.all_reduce(t, "sum", None, "striped" if which == "hier" else "auto")
            torch.cuda.synchronize()
        team.check()
        team.close()
    elif which == "xent":
        from gpubridge_b200.ops.xent import fused_cross_entropy
        logits = (torch.randn(2048, 50304, device=device) * 2).to(torch.bfloat16)
        targets = torch.randint(50257, (2048,), device=device)
        for _ in range(4):
            fused_cross_entropy(logits.clone(), targets, 50257)
        torch.cuda.synchronize()
    elif which == "adamw":
        from gpubridge_b200.ops.optim import FlatAdamW
        p = torch.randn(48 << 20, device=device)
        g = torch.randn(48 << 20, device=device)
        opt = FlatAdamW(p, g)
        for _ in range(4):
            opt.step(zero_grad=False)
        torch.cuda.synchronize()
    elif which == "layernorm":
        from gpubridge_b200.ops.layernorm import FusedLayerNorm
        norm = FusedLayerNorm(768).to(device)
        x = torch.randn(65536, 768, device=device, requires_grad=True)       # 192 MiB
        for _ in range(3):
            y = norm(x)
            y.backward(torch.ones_like(y))
        torch.cuda.synchronize()
    elif which in ("quantize", "dequantize"):
        from gpubridge_b200 import compression as C
        from gpubridge_b200.ops import codec
        n = 64 << 20
        x = torch.randn(n, device=device)
        residual = torch.zeros(n, device=device)
        payload = torch.empty((2, C.payload_nbytes("fp8", n)), dtype=torch.uint8, device=device)
        out = torch.empty(n, device=device)
        codec.quantize("fp8", x, None, payload[1])
        for _ in range(4):
            if which == "quantize":
                codec.quantize("fp8", x, residual, payload[0])
            else:
                codec.dequantize_accumulate("fp8", payload, out)
        torch.cuda.synchronize()
    else:
        raise SystemExit(f"unknown kernel {which!r}")
    print(f"{which}: done")
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv[1] if len(sys.argv) > 1 else "hier"))
