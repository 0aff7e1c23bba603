"""Codec kernel throughput against the device copy bandwidth (the reference's method:
scripts/gpu/bench_compression.py, docs/COMPRESSION.md:228-236).

For each mode, format and dtype: median of ``--trials`` timed launches (CUDA events, after
warm-up, inputs larger than L2) of ``quantize`` (with error feedback, as a training step runs
it) and of ``dequantize_accumulate`` over two members.  Reported as *value* bytes per second
(``numel * element_size / t``, the reference's unit) and as a fraction of what ``b.copy_(a)``
of the same tensor achieves, plus the algorithmic traffic fraction of the measured HBM peak in
``MEASURED_PEAKS.json`` when that file is present.

    python -m gpubridge_b200.bench.bench_compression --numel 268435456 --triton

``--triton`` adds, for every case of the reference's payload format (``ref``), the reference's
own Triton kernels (``baseline/_ref/gpubridge/_compression_kernels.py``, unmodified, compiled by
the Triton in this image on this GPU) timed the same way on the same tensors - the same-box
comparison the kernels here are meant to win.  Those rows carry ``"impl": "reference-triton"``;
when the reference is not installed or Triton cannot compile them, one row says why.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys

import torch

from gpubridge_b200 import compression as C
from gpubridge_b200.ops import codec


def timed(fn, trials: int) -> float:
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    out = []
    for _ in range(trials):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        b.synchronize()
        out.append(a.elapsed_time(b))
    return statistics.median(out)


def reference_triton():
    """The reference's Triton codec module, or a string saying why it cannot be had."""
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    ref = os.path.join(root, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref, "gpubridge")):
        return "baseline/_ref is not installed"
    if ref not in sys.path:
        sys.path.append(ref)
    try:
        from gpubridge import _compression_kernels as kernels
    except Exception as failure:  # noqa: BLE001
        return f"{type(failure).__name__}: {failure}"[:200]
    return kernels


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--numel", type=int, default=1 << 28)
    ap.add_argument("--trials", type=int, default=10)
    ap.add_argument("--dtypes", default="float32,bfloat16")
    ap.add_argument("--only", default="", help="mode:format:dtype:op to run a single case")
    ap.add_argument("--triton", action="store_true",
                    help="also time the reference's Triton kernels on the same tensors")
    args = ap.parse_args(argv)
    n = args.numel
    peaks = {}
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    if os.path.exists(os.path.join(root, "MEASURED_PEAKS.json")):
        peaks = json.load(open(os.path.join(root, "MEASURED_PEAKS.json")))
    rows = []
    triton_kernels = reference_triton() if args.triton else None
    if isinstance(triton_kernels, str):
        rows.append({"impl": "reference-triton", "unavailable": triton_kernels})
        triton_kernels = None
    for dtype_name in args.dtypes.split(","):
        dtype = getattr(torch, dtype_name)
        x = torch.randn(n, device="cuda").to(dtype)
        y = torch.empty_like(x)
        copy_ms = timed(lambda: y.copy_(x), args.trials)
        esize = x.element_size()
        copy_gbs = 2 * n * esize / (copy_ms * 1e-3) / 1e9
        rows.append({"op": "copy", "dtype": dtype_name, "ms": round(copy_ms, 4),
                     "traffic_gbs": round(copy_gbs, 1)})
        for mode in C.MODES:
            if dtype not in C.APPLIES_TO[mode]:
                continue
            for fmt in (C.FORMATS if mode == "fp8" else ("ref",)):
                if args.only and not args.only.startswith(f"{mode}:{fmt}:{dtype_name}"):
                    continue
                nbytes = C.payload_nbytes(mode, n, fmt)
                payload = torch.empty((2, nbytes), dtype=torch.uint8, device="cuda")
                residual = torch.zeros(n, device="cuda")
                out = torch.empty_like(x)
                cases = {
                    "quantize": (lambda: codec.quantize(mode, x, residual, payload[0], fmt),
                                 n * esize + 8 * n + nbytes),          # x, residual r+w, payload
                    "dequantize": (lambda: codec.dequantize_accumulate(mode, payload, out, fmt),
                                   2 * nbytes + n * esize),
                }
                codec.quantize(mode, x, None, payload[1], fmt)
                for op, (fn, traffic) in cases.items():
                    if args.only and not args.only.endswith(op):
                        continue
                    ms = timed(fn, args.trials)
                    row = {"op": op, "mode": mode, "format": fmt, "dtype": dtype_name,
                           "numel": n, "ms": round(ms, 4),
                           "value_gbs": round(n * esize / (ms * 1e-3) / 1e9, 1),
                           "of_copy_value_rate": round((n * esize / ms) / (n * esize / copy_ms), 3),
                           "traffic_gbs": round(traffic / (ms * 1e-3) / 1e9, 1)}
                    if peaks.get("hbm_gbs"):
                        row["traffic_of_measured_hbm"] = round(row["traffic_gbs"] / peaks["hbm_gbs"], 3)
                    rows.append(row)
                if triton_kernels is not None and fmt == "ref":
                    theirs = {
                        "quantize": lambda: triton_kernels.quantize(mode, x, residual, payload[0]),
                        "dequantize": lambda: triton_kernels.dequantize_accumulate(mode, payload, out),
                    }
                    for op, fn in theirs.items():
                        if args.only and not args.only.endswith(op):
                            continue
                        try:
                            ms = timed(fn, args.trials)
                        except Exception as failure:  # noqa: BLE001 - e.g. Triton cannot compile here
                            rows.append({"impl": "reference-triton", "op": op, "mode": mode,
                                         "dtype": dtype_name,
                                         "unavailable": f"{type(failure).__name__}: {failure}"[:200]})
                            continue
                        mine = next(r for r in reversed(rows) if r.get("op") == op and r.get("mode") == mode
                                    and r.get("format") == "ref" and r.get("dtype") == dtype_name
                                    and "impl" not in r)
                        rows.append({"impl": "reference-triton", "op": op, "mode": mode, "format": "ref",
                                     "dtype": dtype_name, "numel": n, "ms": round(ms, 4),
                                     "value_gbs": round(n * esize / (ms * 1e-3) / 1e9, 1),
                                     "of_copy_value_rate": round(copy_ms / ms, 3),
                                     "ours_over_theirs": round(ms / mine["ms"], 3)})
    for row in rows:
        print(json.dumps(row), flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
