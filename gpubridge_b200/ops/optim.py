"""Fused AdamW over flat parameter and gradient buffers (``csrc/gb_optim.cu``)."""
from __future__ import annotations

import torch

from gpubridge_b200.ops import _lib

launches = 0


class FlatAdamW:
    """AdamW whose whole state is three flat float32 buffers and one launch per step.

    Arithmetic is ``torch.optim.AdamW``'s.  The step counter lives on the device and is
    advanced by the kernel, so a step can be captured in a CUDA graph.  ``zero_grad`` makes
    the kernel clear the gradient buffer as it consumes it.
    """

    def __init__(self, flat_param: torch.Tensor, flat_grad: torch.Tensor, lr: float = 1e-3,
                 betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 1e-2) -> None:
        assert flat_param.dtype == torch.float32 and flat_param.is_contiguous()
        assert flat_grad.shape == flat_param.shape and flat_grad.dtype == torch.float32
        self.p, self.g = flat_param, flat_grad
        self.m = torch.zeros_like(flat_param)
        self.v = torch.zeros_like(flat_param)
        self.state = torch.zeros(4, dtype=torch.float32, device=flat_param.device)
        self.lr, self.betas, self.eps, self.weight_decay = lr, betas, eps, weight_decay

    def step(self, grad_scale: float = 1.0, zero_grad: bool = True) -> None:
        self.step_span(0, self.p.numel(), last=True, grad_scale=grad_scale, zero_grad=zero_grad)

    def step_span(self, lo: int, hi: int, last: bool, grad_scale: float = 1.0,
                  zero_grad: bool = True, max_blocks: int = 0) -> None:
        """Update elements ``[lo, hi)`` (``lo`` a multiple of 4) as a part of the step in
        progress.  The parts of a step are launched in stream order; the one launched last
        passes ``last=True`` and advances the step count.  ``max_blocks`` caps the grid of a
        part that runs beside other kernels."""
        global launches
        if self.p.device.type != "cuda":
            self._reference_step(grad_scale, zero_grad, lo, hi, last)
            return
        assert lo % 4 == 0
        code = _lib.lib().gb_adamw_span(
            self.p.data_ptr() + 4 * lo, self.g.data_ptr() + 4 * lo, self.m.data_ptr() + 4 * lo,
            self.v.data_ptr() + 4 * lo, hi - lo, self.state.data_ptr(), self.lr, self.betas[0],
            self.betas[1], self.eps, self.weight_decay, grad_scale, int(zero_grad), int(last),
            int(max_blocks), _lib.stream_ptr(self.p.device))
        _lib.check(code, "gb_adamw_span")
        launches += 1

    def _reference_step(self, grad_scale: float, zero_grad: bool, lo: int = 0, hi: int | None = None,
                        last: bool = True) -> None:
        """The same update in plain PyTorch (CPU runs and the oracle of the kernel test)."""
        hi = self.p.numel() if hi is None else hi
        step = float(self.state[2]) + 1
        if last:
            self.state[2] += 1
        b1, b2 = self.betas
        p, m, v = self.p[lo:hi], self.m[lo:hi], self.v[lo:hi]
        g = self.g[lo:hi] * grad_scale
        p.mul_(1 - self.lr * self.weight_decay)
        m.mul_(b1).add_(g, alpha=1 - b1)
        v.mul_(b2).addcmul_(g, g, value=1 - b2)
        denom = (v.sqrt() / (1 - b2 ** step) ** 0.5).add_(self.eps)
        p.addcdiv_(m, denom, value=-self.lr / (1 - b1 ** step))
        if zero_grad:
            self.g[lo:hi].zero_()
