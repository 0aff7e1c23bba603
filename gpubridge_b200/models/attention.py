"""Causal attention for the benchmark models: ``F.scaled_dot_product_attention`` with the
backend chosen by ``GPUBRIDGE_SDPA`` - ``auto`` (torch's own choice, the default), ``cudnn``
(cuDNN's fused attention first, then flash), ``flash``, ``efficient`` or ``math``.  The
reference's models call ``F.scaled_dot_product_attention(is_causal=True)`` and leave the choice
to torch (scripts/gpu/llama.py:109, train_bench.py:172); this keeps that default and makes the
choice measurable."""
from __future__ import annotations

import functools
import os

import torch
import torch.nn.functional as F


@functools.lru_cache(maxsize=None)
def _backends(choice: str):
    if choice in ("", "auto"):
        return None
    from torch.nn.attention import SDPBackend
    table = {"cudnn": [SDPBackend.CUDNN_ATTENTION, SDPBackend.FLASH_ATTENTION,
                       SDPBackend.EFFICIENT_ATTENTION, SDPBackend.MATH],
             "flash": [SDPBackend.FLASH_ATTENTION, SDPBackend.EFFICIENT_ATTENTION, SDPBackend.MATH],
             "efficient": [SDPBackend.EFFICIENT_ATTENTION, SDPBackend.MATH],
             "math": [SDPBackend.MATH]}
    if choice not in table:
        raise ValueError(f"GPUBRIDGE_SDPA must be auto, cudnn, flash, efficient or math, got {choice!r}")
    return table[choice]


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, **kwargs) -> torch.Tensor:
    backends = _backends(os.environ.get("GPUBRIDGE_SDPA", "auto").strip().lower())
    if backends is None or not q.is_cuda:
        return F.scaled_dot_product_attention(q, k, v, is_causal=True, **kwargs)
    from torch.nn.attention import sdpa_kernel
    try:
        context = sdpa_kernel(backends, set_priority=True)
    except TypeError:                       # older torch: no priority order
        context = sdpa_kernel(backends)
    with context:
        return F.scaled_dot_product_attention(q, k, v, is_causal=True, **kwargs)
