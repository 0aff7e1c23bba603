"""sm_100a codec kernels: quantise into / dequantise-accumulate out of the bridge payload.

Same arguments and same bits as :func:`gpubridge_b200.compression.quantize_reference` and
:func:`~gpubridge_b200.compression.dequantize_accumulate_reference`; these replace the
reference's Triton kernels (src/gpubridge/_compression_kernels.py:116-226) with kernels in
``csrc/gb_codec.cu`` that use the hardware fp8 conversion.
"""
from __future__ import annotations

import torch

from gpubridge_b200.ops import _lib

_MODES = {"bf16": 0, "fp8": 1}
_FORMATS = {"ref": 0, "b200": 1}
launches = 0     # kernels launched through this module


def quantize(mode: str, x: torch.Tensor, residual: torch.Tensor | None, payload: torch.Tensor,
             fmt: str = "ref") -> None:
    global launches
    if not x.is_contiguous() or not payload.is_contiguous():
        raise ValueError("codec tensors must be contiguous")
    if residual is not None and (residual.dtype != torch.float32 or residual.numel() != x.numel()):
        raise ValueError("the residual must be float32 with one value per element")
    L = _lib.lib()
    code = L.gb_codec_quantize(_MODES[mode], _FORMATS[fmt], _lib.DTYPES[x.dtype], x.data_ptr(),
                               residual.data_ptr() if residual is not None else None,
                               payload.data_ptr(), x.numel(), _lib.stream_ptr(x.device))
    _lib.check(code, "gb_codec_quantize")
    launches += 1


def dequantize_accumulate(mode: str, payloads: torch.Tensor, out: torch.Tensor,
                          fmt: str = "ref") -> None:
    global launches
    if payloads.dim() != 2 or payloads.stride(1) != 1 or not out.is_contiguous():
        raise ValueError("payloads must be a (members, bytes) tensor with contiguous rows")
    L = _lib.lib()
    code = L.gb_codec_dequantize(_MODES[mode], _FORMATS[fmt], _lib.DTYPES[out.dtype],
                                 payloads.data_ptr(), payloads.stride(0), payloads.shape[0],
                                 out.data_ptr(), out.numel(), _lib.stream_ptr(out.device))
    _lib.check(code, "gb_codec_dequantize")
    launches += 1
