"""Where a codec implementation differs from the oracle, value by value.

    python -m gpubridge_b200.kit.codec_diagnosis [--mode fp8] [--format ref] [--numel 70001] [--device cuda]

The codec kernels must produce the oracle's bits (:mod:`gpubridge_b200.compression`:
``quantize_reference``).  When a test says they do not, this program reruns one case - awkward
inputs (huge, tiny, subnormal, non-finite, cancelling values), a prior residual - through the
implementation under test and through the oracle, and for the first values whose payload byte,
scale or new residual differs prints what each step computed: the input, the prior residual,
``v`` (input plus residual in float32, tiny flushed), the block's largest magnitude, the stored
scale, the code and what it decodes to, what was sent, both residuals with their bits, and what
a fused multiply-add would have given for ``v - decoded * scale`` (one rounding instead of two:
the usual culprit).  Exit code 0 when nothing differs.  Without a GPU the implementation under
test is the oracle's own dispatch on CPU.  (Reference: scripts/gpu/diag_fp8_residual.py.)
"""
from __future__ import annotations

import argparse
import math
import sys

import torch

from gpubridge_b200 import compression as C


def awkward(n: int, seed: int = 5) -> tuple[torch.Tensor, torch.Tensor]:
    """(values, prior residual): every regime of the codec in one tensor."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(n, generator=g) * torch.exp(torch.randn(n, generator=g) * 6)
    x[::97] = 0.0
    x[1::193] = 3e38
    x[2::211] = 1e-40
    x[3::223] = 2.0 ** -101
    if n > 5:
        x[4], x[5] = float("inf"), float("nan")
    residual = torch.randn(n, generator=g) * 1e-3
    return x, residual


def bits(value: float) -> str:
    return f"0x{torch.tensor([value], dtype=torch.float32).view(torch.int32).item() & 0xFFFFFFFF:08x}"


def run(quantize, mode: str, fmt: str, x: torch.Tensor, residual: torch.Tensor, device: str):
    payload = torch.zeros(C.payload_nbytes(mode, x.numel(), fmt), dtype=torch.uint8, device=device)
    kept = residual.clone().to(device)
    quantize(mode, x.to(device), kept, payload, fmt)
    return payload.cpu(), kept.cpu()


def differences(mode: str, fmt: str, x, prior, got, want, limit: int = 8) -> list[str]:
    """Text for the first ``limit`` values where (payload, residual) ``got`` differs from ``want``."""
    n = x.numel()
    payload, residual = got
    ref_payload, ref_residual = want
    size, nb = C.block_size(fmt), C.n_blocks(n, fmt)
    head = 4 * nb if mode == "fp8" else 0
    width = 1 if mode == "fp8" else 2
    codes = payload[head:head + width * n].view(n, width)
    ref_codes = ref_payload[head:head + width * n].view(n, width)
    wrong_code = (codes != ref_codes).any(dim=1)
    same_residual = (residual.view(torch.int32) == ref_residual.view(torch.int32)) | (residual.isnan() & ref_residual.isnan())
    where = torch.nonzero(wrong_code | ~same_residual).flatten().tolist()
    lines = []
    if mode == "fp8" and not torch.equal(payload[:head], ref_payload[:head]):
        scales, ref_scales = payload[:head].view(torch.float32), ref_payload[:head].view(torch.float32)
        for b in torch.nonzero(scales != ref_scales).flatten().tolist()[:limit]:
            lines.append(f"block {b}: scale {float(scales[b])!r} ({bits(float(scales[b]))}), "
                         f"oracle {float(ref_scales[b])!r} ({bits(float(ref_scales[b]))})")
    v, finite = C.prepare(x, prior)
    for i in where[:limit]:
        block = i // size
        lo, hi = block * size, min(n, (block + 1) * size)
        amax = float(torch.where(finite[lo:hi], v[lo:hi], torch.zeros(hi - lo)).abs().max())
        line = [f"value {i} (block {block}): input {float(x[i])!r}, prior residual {float(prior[i])!r}, "
                f"v {float(v[i])!r} ({bits(float(v[i]))}), block amax {amax!r}"]
        if mode == "fp8":
            scale = float(ref_payload[:head].view(torch.float32)[block])
            decoded, ref_decoded = float(C.e4m3_decode(codes[i])[0]), float(C.e4m3_decode(ref_codes[i])[0])
            line.append(f"  scale {scale!r}; code 0x{int(codes[i][0]):02x} -> {decoded!r}, oracle 0x{int(ref_codes[i][0]):02x} -> {ref_decoded!r}")
            if math.isfinite(ref_decoded) and math.isfinite(float(v[i])):
                fused = math.fma(-ref_decoded, scale, float(v[i])) if hasattr(math, "fma") else float("nan")
                line.append(f"  sent {ref_decoded * scale!r}; a fused multiply-add would leave {fused!r} ({bits(fused)})")
        else:
            line.append(f"  code 0x{int(codes[i].view(torch.int16)) & 0xFFFF:04x}, oracle 0x{int(ref_codes[i].view(torch.int16)) & 0xFFFF:04x}")
        line.append(f"  residual {float(residual[i])!r} ({bits(float(residual[i]))}), oracle {float(ref_residual[i])!r} ({bits(float(ref_residual[i]))})"
                    + ("  [subnormal]" if 0 < abs(float(ref_residual[i])) < torch.finfo(torch.float32).tiny else ""))
        lines.append("\n".join(line))
    if len(where) > limit:
        lines.append(f"... and {len(where) - limit} more values differ")
    return lines


def diagnose(mode: str, fmt: str, numel: int, device: str, quantize=None) -> list[str]:
    x, prior = awkward(numel)
    want = run(C.quantize_reference, mode, fmt, x, prior, "cpu")
    got = run(quantize or C.quantize, mode, fmt, x, prior, device)
    return differences(mode, fmt, x, prior, got, want)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--mode", default="fp8", choices=C.MODES)
    ap.add_argument("--format", default="ref", choices=C.FORMATS)
    ap.add_argument("--numel", type=int, default=70_001)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    args = ap.parse_args(argv)
    found = diagnose(args.mode, args.format, args.numel, args.device)
    for text in found:
        print(text)
    print(f"{args.mode}/{args.format} on {args.device}: " + ("identical to the oracle" if not found else "DIFFERS from the oracle"))
    return 1 if found else 0


if __name__ == "__main__":
    sys.exit(main())
