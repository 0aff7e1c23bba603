"""Fused LayerNorm (``csrc/gb_layernorm.cu``): one warp per row, the output written once in the
dtype the consumer wants, dx and the gamma / beta partial sums in one backward pass.

``FusedLayerNorm`` is an ``nn.LayerNorm`` (same parameters, same state dict) whose forward uses
the kernels for CUDA inputs of width 128 k (k = 1..8, 10, 12, 16) and ``F.layer_norm`` otherwise;
``GPUBRIDGE_FUSED_NORM=0`` switches the kernels off.  Under ``torch.autocast`` the output is the
autocast dtype: ``F.layer_norm`` would produce fp32 and the next Linear would cast it, which is
the same rounding done by one more kernel.
"""
from __future__ import annotations

import os

import torch
import torch.nn.functional as F
from torch import nn

from gpubridge_b200.ops import _lib

launches = 0
_WIDTHS = frozenset(128 * k for k in (1, 2, 3, 4, 5, 6, 7, 8, 10, 12, 16))
_CODES = {torch.float32: 0, torch.bfloat16: 1}


def enabled() -> bool:
    return os.environ.get("GPUBRIDGE_FUSED_NORM", "1") != "0"


def usable(x: torch.Tensor, weight: torch.Tensor | None, bias: torch.Tensor | None) -> bool:
    return (x.is_cuda and x.dtype in _CODES and x.shape[-1] in _WIDTHS and weight is not None
            and bias is not None and weight.dtype == torch.float32 and x.numel() > 0)


def _declare(lib):
    if getattr(lib, "_ln_declared", False):
        return lib
    import ctypes
    vp, i, f, lg = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_long
    lib.gb_layernorm_fwd.argtypes = [i, i, vp, vp, vp, vp, vp, vp, lg, i, f, vp]
    lib.gb_layernorm_bwd.argtypes = [i, i, vp, vp, vp, vp, vp, vp, vp, vp, vp, lg, i, vp]
    lib.gb_layernorm_scratch.argtypes = [lg, i]
    lib.gb_layernorm_scratch.restype = lg
    lib._ln_declared = True
    return lib


class _LayerNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, eps, out_dtype):
        global launches
        lib = _declare(_lib.lib())
        d = x.shape[-1]
        x2 = x.reshape(-1, d)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        rows = x2.shape[0]
        if x2.dtype == torch.bfloat16:
            out_dtype = torch.bfloat16
        y = torch.empty((rows, d), dtype=out_dtype, device=x.device)
        mean = torch.empty(rows, dtype=torch.float32, device=x.device)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        stream = torch.cuda.current_stream(x.device).cuda_stream
        _lib.check(lib.gb_layernorm_fwd(_CODES[x2.dtype], _CODES[out_dtype], x2.data_ptr(),
                                        weight.data_ptr(), bias.data_ptr(), y.data_ptr(),
                                        mean.data_ptr(), rstd.data_ptr(), rows, d, float(eps), stream),
                   "gb_layernorm_fwd")
        launches += 1
        ctx.save_for_backward(x2, weight, mean, rstd)
        ctx.shape = x.shape
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        global launches
        lib = _declare(_lib.lib())
        x2, weight, mean, rstd = ctx.saved_tensors
        rows, d = x2.shape
        dy2 = dy.reshape(rows, d)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        if dy2.dtype not in _CODES or (x2.dtype == torch.bfloat16 and dy2.dtype != torch.bfloat16):
            dy2 = dy2.to(x2.dtype)
        dx = torch.empty_like(x2)
        part = torch.empty(lib.gb_layernorm_scratch(rows, d), dtype=torch.float32, device=x2.device)
        dgamma = torch.empty(d, dtype=torch.float32, device=x2.device)
        dbeta = torch.empty(d, dtype=torch.float32, device=x2.device)
        stream = torch.cuda.current_stream(x2.device).cuda_stream
        _lib.check(lib.gb_layernorm_bwd(_CODES[x2.dtype], _CODES[dy2.dtype], dy2.data_ptr(),
                                        x2.data_ptr(), weight.data_ptr(), mean.data_ptr(),
                                        rstd.data_ptr(), dx.data_ptr(), part.data_ptr(),
                                        dgamma.data_ptr(), dbeta.data_ptr(), rows, d, stream),
                   "gb_layernorm_bwd")
        launches += 2
        return dx.view(ctx.shape), dgamma, dbeta, None, None


def fused_layer_norm(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor,
                     eps: float = 1e-5) -> torch.Tensor:
    """LayerNorm over the last dimension; see the module docstring for dtypes."""
    out_dtype = x.dtype
    if x.dtype == torch.float32 and torch.is_autocast_enabled():
        out_dtype = (torch.get_autocast_dtype("cuda") if hasattr(torch, "get_autocast_dtype")
                     else torch.get_autocast_gpu_dtype())
        if out_dtype not in _CODES:
            out_dtype = torch.float32
    return _LayerNorm.apply(x, weight, bias, eps, out_dtype)


class FusedLayerNorm(nn.LayerNorm):
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if (enabled() and len(self.normalized_shape) == 1
                and usable(x, self.weight, self.bias)):
            return fused_layer_norm(x, self.weight, self.bias, self.eps)
        return F.layer_norm(x, self.normalized_shape, self.weight, self.bias, self.eps)
