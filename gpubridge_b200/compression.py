"""Bridge compression: bf16 and block-scaled fp8-e4m3 with error feedback.

Numerics are the reference's (src/gpubridge/compression.py:64-261, docs/COMPRESSION.md):
only floating-point SUM/AVG on the bridge step is compressed; every member's payload is
exchanged *once* and never re-quantised, payloads are dequantised and added in fp32 in
member order with magnitudes below ``TINY`` flushed after every add, then rounded once to
the output dtype - so every rank of every island ends with identical bits and the error
does not compound with the island count.  Error feedback keeps, per buffer, what the last
payload left out (``v - sent``) and adds it to the next call's values.

Two payload formats:

``ref``   the reference's, bit for bit: 256 values per block, power-of-two scale
          (smallest 2^k with amax/2^k <= 448, k <= 119, 0 for an all-zero block);
          payload = fp32 scales, then one code byte per value, padded to 4 bytes.
``b200``  128 values per block, fp32 scale ``amax/448`` (the format of the HSDP benchmark);
          same layout with 128-value blocks.  Encoding multiplies by ``448/amax``.

Per-quantisation error bounds (the numerical gate): bf16 ``2^-8 |v|``; fp8
``2^-4 |v| + 2^-10 s`` with ``s`` the block scale.

This module is the plain-PyTorch codec (the oracle, and what CPU simulation runs).  On a
GPU :func:`quantize` / :func:`dequantize_accumulate` dispatch to the sm_100a kernels of
:mod:`gpubridge_b200.ops.codec`, and the fused collectives quantise inside the reducing
kernel; all three produce the same bits.
"""
from __future__ import annotations

import threading
import weakref
from collections.abc import Callable, Sequence
from typing import TYPE_CHECKING

import torch

from gpubridge_b200.observe import phase

if TYPE_CHECKING:
    from gpubridge_b200.transport import BridgeTransport

BLOCK = 256                 # values per scale, ``ref`` format
BLOCK_B200 = 128            # values per scale, ``b200`` format
FP8_MAX = 448.0
FLT_MAX = torch.finfo(torch.float32).max
MAX_SCALE_EXP = 119         # 448 * 2^119 is the largest code*scale float32 holds
TINY = 2.0 ** -100          # magnitudes below this count as zero

APPLIES_TO: dict[str, frozenset[torch.dtype]] = {
    "bf16": frozenset({torch.float32, torch.float64}),
    "fp8": frozenset({torch.float16, torch.bfloat16, torch.float32, torch.float64}),
}
MODES = tuple(APPLIES_TO)
FORMATS = ("ref", "b200")


def applies(mode: str | None, dtype: torch.dtype) -> bool:
    return bool(mode) and dtype in APPLIES_TO[mode]  # type: ignore[index]


def block_size(fmt: str) -> int:
    return BLOCK if fmt == "ref" else BLOCK_B200


def _ceil_to(n: int, m: int) -> int:
    return -(-n // m) * m


def n_blocks(numel: int, fmt: str = "ref") -> int:
    return -(-numel // block_size(fmt))


def payload_nbytes(mode: str, numel: int, fmt: str = "ref") -> int:
    """Bytes one member sends for ``numel`` values (always a multiple of 4)."""
    if mode == "bf16":
        return _ceil_to(2 * numel, 4)
    return 4 * n_blocks(numel, fmt) + _ceil_to(numel, 4)


# ---- scalar building blocks, vectorised over tensors ------------------------------------

def _e4m3_table(device) -> torch.Tensor:
    """All 256 code values as float32 (0x7F and 0xFF are NaN)."""
    codes = torch.arange(256, dtype=torch.int32, device=device).to(torch.uint8)
    table = codes.view(torch.float8_e4m3fn).to(torch.float32)
    table[0x7F] = table[0xFF] = float("nan")      # one canonical quiet NaN (0x7FC00000)
    return table


def e4m3_decode(codes: torch.Tensor) -> torch.Tensor:
    """float32 value of each uint8 E4M3 code."""
    return _e4m3_table(codes.device)[codes.to(torch.int64)]


def e4m3_encode(q: torch.Tensor) -> torch.Tensor:
    """uint8 E4M3 codes of finite float32 ``q``: round to nearest even, |q| > 448
    saturates, a zero (of either sign) encodes as 0x00."""
    clipped = q.clamp(-FP8_MAX, FP8_MAX)
    codes = clipped.to(torch.float8_e4m3fn).view(torch.uint8)
    return torch.where(q == 0, torch.zeros_like(codes), codes)


def bf16_bits(v: torch.Tensor) -> torch.Tensor:
    """int32 bfloat16 bit patterns (0..0xFFFF) of float32 ``v``, nearest even; NaN 0x7FC0."""
    bits = v.contiguous().view(torch.int32)
    rounded = ((bits + (0x7FFF + ((bits >> 16) & 1))) >> 16) & 0xFFFF
    return torch.where(torch.isnan(v), torch.full_like(rounded, 0x7FC0), rounded)


def bf16_codes(v: torch.Tensor) -> torch.Tensor:
    """:func:`bf16_bits`, but a finite value that would round to +-inf keeps the largest
    finite bfloat16 instead."""
    bits = bf16_bits(v)
    return torch.where((bits & 0x7FFF) == 0x7F80, bits - 1, bits)


def _from_bf16_bits(bits: torch.Tensor) -> torch.Tensor:
    return (bits.to(torch.int32) << 16).view(torch.float32)


def prepare(x: torch.Tensor, residual: torch.Tensor | None) -> tuple[torch.Tensor, torch.Tensor]:
    """``x (+ residual)`` as float32, saturated to float32's finite range, tiny values
    zeroed; and the mask of values that are finite (in ``x``'s dtype and after the add)."""
    flat = x.reshape(-1)
    finite = torch.isfinite(flat)
    v = flat.to(torch.float32)
    v = torch.where(finite, v.clamp(-FLT_MAX, FLT_MAX), v)
    if residual is not None:
        v = v + residual
        v = torch.where(finite, v.clamp(-FLT_MAX, FLT_MAX), v)
    finite = finite & ~v.isnan()
    v = torch.where(finite & (v.abs() < TINY), torch.zeros_like(v), v)
    return v, finite


def pow2_scale_exponent(amax: torch.Tensor) -> torch.Tensor:
    """k of the ``ref`` scale 2^k.  With amax = m * 2^e, m in [0.5, 1): 448 = 0.875 * 2^9,
    so k = e - 9, one more when m > 0.875."""
    mant, exp = torch.frexp(amax)
    k = exp.to(torch.int32) - 9 + (mant > 0.875).to(torch.int32)
    k = k.clamp(max=MAX_SCALE_EXP)
    return torch.where(amax == 0, torch.zeros_like(k), k)


def _exp2(k: torch.Tensor) -> torch.Tensor:
    return ((k.to(torch.int32) + 127) << 23).view(torch.float32)


def block_scales(blocks: torch.Tensor, fmt: str) -> tuple[torch.Tensor, torch.Tensor]:
    """(scale, multiplier) per row of ``blocks``: the stored scale and what values are
    multiplied by before encoding."""
    amax = blocks.abs().amax(dim=1)
    if fmt == "ref":
        k = pow2_scale_exponent(amax)
        return _exp2(k), _exp2(-k)
    # Both quotients must be correctly rounded divisions (what the kernels compute):
    # ``scalar / tensor`` is evaluated by torch as ``tensor.reciprocal() * scalar``.
    one = torch.ones_like(amax)
    top = torch.full_like(amax, FP8_MAX)
    safe = torch.where(amax == 0, one, amax)
    scale = torch.where(amax == 0, one, safe / top)
    mult = torch.where(amax == 0, one, top / safe)
    return scale, mult


# ---- the codec ----------------------------------------------------------------------------

def quantize_reference(mode: str, x: torch.Tensor, residual: torch.Tensor | None,
                       payload: torch.Tensor, fmt: str = "ref") -> None:
    """Compress ``x`` (+ ``residual``) into the uint8 ``payload`` (padding zeroed) and leave
    the new residual: what the payload leaves out of each finite value, 0 elsewhere."""
    n = x.numel()
    v, finite = prepare(x, residual)
    if mode == "bf16":
        bits = torch.where(finite, bf16_codes(v), bf16_bits(v))
        payload[:2 * n].view(torch.int16).copy_(bits.to(torch.int16))
        payload[2 * n:].zero_()
        sent = _from_bf16_bits(bits)
    elif mode == "fp8":
        size, nb = block_size(fmt), n_blocks(n, fmt)
        padded = torch.zeros(nb * size, dtype=torch.float32, device=v.device)
        padded[:n] = torch.where(finite, v, torch.zeros_like(v))
        blocks = padded.view(nb, size)
        scale, mult = block_scales(blocks, fmt)
        q = (blocks * mult[:, None]).view(-1)[:n]
        codes = torch.where(finite, e4m3_encode(q), torch.full_like(q, 0x7F, dtype=torch.uint8))
        payload[:4 * nb].view(torch.float32).copy_(scale)
        payload[4 * nb:4 * nb + n].copy_(codes)
        payload[4 * nb + n:].zero_()
        sent = e4m3_decode(codes) * scale.repeat_interleave(size)[:n]
    else:
        raise ValueError(f"unknown compression mode {mode!r}")
    if residual is not None:
        residual.copy_(torch.where(finite, v - sent, torch.zeros_like(v)))


def dequantize_row(mode: str, row: torch.Tensor, n: int, fmt: str = "ref") -> torch.Tensor:
    if mode == "bf16":
        return _from_bf16_bits(row[:2 * n].view(torch.int16).to(torch.int32) & 0xFFFF)
    size, nb = block_size(fmt), n_blocks(n, fmt)
    scale = row[:4 * nb].view(torch.float32)
    return e4m3_decode(row[4 * nb:4 * nb + n]) * scale.repeat_interleave(size)[:n]


def dequantize_accumulate_reference(mode: str, payloads: torch.Tensor, out: torch.Tensor,
                                    fmt: str = "ref", scale: float | None = None) -> None:
    """Sum the rows of ``payloads`` into ``out`` in row order (fp32, tiny flushed after every
    add), divide by ``scale`` if given (the fused AVG), round once to ``out``'s dtype."""
    n = out.numel()
    acc = torch.zeros(n, dtype=torch.float32, device=out.device)
    for row in payloads:
        acc = acc + dequantize_row(mode, row, n, fmt)
        acc = torch.where(acc.abs() < TINY, torch.zeros_like(acc), acc)
    if scale is not None:
        acc = acc / scale
    if out.dtype == torch.bfloat16:
        out.view(-1).view(torch.int16).copy_(bf16_bits(acc).to(torch.int16))
    else:
        out.view(-1).copy_(acc.to(out.dtype))


def error_bound(mode: str, v: torch.Tensor, fmt: str = "ref") -> torch.Tensor:
    """The per-value bound on ``|v - sent|`` of one quantisation of float32 ``v``."""
    v = v.reshape(-1).to(torch.float32)
    if mode == "bf16":
        return v.abs() * 2.0 ** -8
    size, nb = block_size(fmt), n_blocks(v.numel(), fmt)
    padded = torch.zeros(nb * size)
    padded[:v.numel()] = v
    scale, _ = block_scales(padded.view(nb, size), fmt)
    return v.abs() * 2.0 ** -4 + scale.repeat_interleave(size)[:v.numel()] * 2.0 ** -10


# ---- dispatch ------------------------------------------------------------------------------

KERNELS_ENV = "GPUBRIDGE_COMPRESSION_KERNELS"


def kernels_setting() -> str:
    """``auto`` (default): the sm_100a kernels on GPU tensors, PyTorch otherwise; ``native``:
    the kernels or an error; ``torch``: the PyTorch codec everywhere (the reference's values
    are auto | triton | torch, compression.py:89 there; ``triton`` is read as ``native``)."""
    import os
    value = os.environ.get(KERNELS_ENV, "auto").strip().lower() or "auto"
    if value == "triton":
        value = "native"
    if value not in ("auto", "native", "torch"):
        raise ValueError(f"{KERNELS_ENV} must be auto, native or torch, got {value!r}")
    return value


def _device_codec(tensor: torch.Tensor):
    choice = kernels_setting()
    if choice == "torch":
        return None
    if tensor.device.type != "cuda":
        if choice == "native":
            raise RuntimeError(f"{KERNELS_ENV}=native: the codec kernels need a CUDA tensor, "
                               f"got one on {tensor.device}")
        return None
    from gpubridge_b200.ops import codec
    return codec


def quantize(mode: str, x: torch.Tensor, residual: torch.Tensor | None,
             payload: torch.Tensor, fmt: str = "ref") -> None:
    kernels = _device_codec(x)
    if kernels is None:
        quantize_reference(mode, x, residual, payload, fmt)
    else:
        kernels.quantize(mode, x, residual, payload, fmt)


def dequantize_accumulate(mode: str, payloads: torch.Tensor, out: torch.Tensor,
                          fmt: str = "ref") -> None:
    kernels = _device_codec(out)
    if kernels is None:
        dequantize_accumulate_reference(mode, payloads, out, fmt)
    else:
        kernels.dequantize_accumulate(mode, payloads, out, fmt)


# ---- error feedback state and the host-staged exchange ---------------------------------------

def buffer_key(tensor: torch.Tensor, part: int = 0) -> tuple:
    """Error feedback finds a buffer's residual by device, address, size, dtype and part."""
    return (str(tensor.device), tensor.data_ptr(), tensor.numel(), tensor.dtype, part)


_compressors: "weakref.WeakSet[BridgeCompressor]" = weakref.WeakSet()


def reset_error_feedback() -> None:
    """Forget every residual on this rank (call after reallocating gradient buffers)."""
    for compressor in list(_compressors):
        compressor.reset()


class BridgeCompressor:
    """One bridge member's compression state and its side of a compressed bridge step."""

    def __init__(self, mode: str, fmt: str = "ref") -> None:
        if mode not in MODES:
            raise ValueError(f"unknown bridge compression mode {mode!r}; use one of "
                             f"{', '.join(MODES)}")
        if fmt not in FORMATS:
            raise ValueError(f"unknown codec format {fmt!r}; use one of {', '.join(FORMATS)}")
        self.mode, self.fmt = mode, fmt
        self._residuals: dict[tuple, torch.Tensor] = {}
        self._lock = threading.Lock()
        _compressors.add(self)

    def applies(self, dtype: torch.dtype) -> bool:
        return applies(self.mode, dtype)

    def residual(self, key: tuple, like: torch.Tensor) -> torch.Tensor:
        with self._lock:
            kept = self._residuals.get(key)
            if kept is None or kept.numel() != like.numel() or kept.device != like.device:
                kept = self._residuals[key] = torch.zeros(like.numel(), dtype=torch.float32,
                                                          device=like.device)
            return kept

    def reset(self) -> None:
        with self._lock:
            self._residuals.clear()

    def compress(self, segment: torch.Tensor, key: tuple, members: Sequence[int],
                 me: int) -> torch.Tensor:
        rows = torch.empty((len(members), payload_nbytes(self.mode, segment.numel(), self.fmt)),
                           dtype=torch.uint8, device=segment.device)
        with phase("compress"):
            quantize(self.mode, segment, self.residual(key, segment), rows[me], self.fmt)
        return rows

    def decompress(self, rows: torch.Tensor, segment: torch.Tensor) -> None:
        with phase("decompress"):
            dequantize_accumulate(self.mode, rows, segment, self.fmt)

    def all_reduce(self, segment: torch.Tensor, key: tuple, bridge: "BridgeTransport",
                   members: Sequence[int], *, rank: int, direct: bool = False) -> None:
        """Replace ``segment`` (this member's island sum) by the sum of every member's,
        compressed: quantise, every member broadcasts its payload in turn, dequantise."""
        me = list(members).index(rank)
        rows = self.compress(segment, key, members, me)
        with phase("bridge"):
            staged = rows if direct else host_rows(rows, me)
            for i, src in enumerate(members):
                bridge.broadcast(staged[i], src=src)
            if staged is not rows:
                for i in range(len(members)):
                    if i != me:
                        rows[i].copy_(staged[i])
        self.decompress(rows, segment)


def _host_rows(rows: torch.Tensor, me: int) -> torch.Tensor:
    if rows.device.type == "cpu":
        return rows
    host = torch.empty(rows.shape, dtype=rows.dtype)
    host[me].copy_(rows[me])
    return host


#: Tests replace this with one that always copies, to run the GPU path's copies on CPU.
host_rows: Callable[[torch.Tensor, int], torch.Tensor] = _host_rows
