"""Fused softmax cross-entropy (``csrc/gb_xent.cu``): the mean loss and, in the same
launch, its gradient written over the logits."""
from __future__ import annotations

import torch
import torch.nn.functional as F

from gpubridge_b200.ops import _lib

launches = 0
_scratch: dict[tuple, tuple[torch.Tensor, torch.Tensor]] = {}


def _get_scratch(device: torch.device, rows: int) -> tuple[torch.Tensor, torch.Tensor]:
    key = (device.type, device.index)
    kept = _scratch.get(key)
    if kept is None or kept[0].numel() < rows:
        kept = (torch.empty(rows, dtype=torch.float32, device=device),
                torch.zeros(1, dtype=torch.int32, device=device))
        _scratch[key] = kept
    return kept


class _FusedCrossEntropy(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits: torch.Tensor, targets: torch.Tensor, vocab: int, unit_grad: bool):
        global launches
        rows, ld = logits.shape
        row_loss, counter = _get_scratch(logits.device, rows)
        loss = torch.empty((), dtype=torch.float32, device=logits.device)
        code = _lib.lib().gb_xent_fwd_bwd(
            logits.data_ptr(), 1 if logits.dtype == torch.bfloat16 else 0, targets.data_ptr(),
            rows, vocab, ld, row_loss.data_ptr(), counter.data_ptr(), loss.data_ptr(),
            _lib.stream_ptr(logits.device))
        _lib.check(code, "gb_xent_fwd_bwd")
        launches += 1
        ctx.mark_dirty(logits)                 # now holds d(loss)/d(logits)
        ctx.save_for_backward(logits)
        ctx.unit_grad = unit_grad
        ctx.mark_non_differentiable(logits)
        return loss, logits                    # a tensor modified in place must be an output

    @staticmethod
    def backward(ctx, grad_loss, _unused=None):
        (grad_logits,) = ctx.saved_tensors
        if not ctx.unit_grad:
            grad_logits = grad_logits * grad_loss.to(grad_logits.dtype)
        return grad_logits, None, None, None


def fused_cross_entropy(logits: torch.Tensor, targets: torch.Tensor, vocab: int | None = None,
                        unit_grad: bool = False) -> torch.Tensor:
    """Mean cross-entropy of ``logits[:, :vocab]`` against ``targets``.

    ``logits`` is a contiguous ``[rows, ld]`` bf16 or fp32 matrix that nothing else reads
    afterwards: it is **overwritten** with the gradient (columns at or past ``vocab`` get
    zero).  ``unit_grad=True`` promises that backward starts at this loss
    (``loss.backward()``), which saves one pass that would scale the stored gradient.
    Falls back to ``F.cross_entropy`` off the GPU.
    """
    vocab = logits.shape[-1] if vocab is None else vocab
    usable = (logits.is_cuda and logits.dim() == 2 and logits.is_contiguous()
              and logits.dtype in (torch.bfloat16, torch.float32)
              and logits.shape[1] % (8 if logits.dtype == torch.bfloat16 else 4) == 0
              and logits.data_ptr() % 16 == 0 and targets.dtype == torch.int64
              and targets.is_contiguous())
    if not usable:
        return F.cross_entropy(logits[:, :vocab].float(), targets)
    return _FusedCrossEntropy.apply(logits, targets, vocab, unit_grad)[0]
