"""Next-token cross-entropy for the training step: loss and logit gradient in one pass over the bf16 logits
(C ABI ``wkv6_softmax_xent_bf16``).  ``lm_loss(logits, targets)`` equals
``torch.nn.functional.cross_entropy(logits.float().view(-1, V), targets.view(-1))`` (mean over all tokens) and its
gradient when every target lies in [0, V); a row whose target lies outside that range contributes zero loss and zero
gradient and still counts in the mean's denominator (on both the fused path and the library path), without the fp32 copy of the logits, the stored log-probabilities and the separate backward pass.

The gradient is written over the logits inside the forward call: the logits tensor must not be used afterwards
(the output layer's own backward needs only its input, so a model may pass its logits straight in).
"""
from __future__ import annotations

import torch

from ._lib import check, lib
from .ops import _check_cuda, _ptr, _stream


class _LMLoss(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, targets):
        V = logits.shape[-1]
        z = logits.detach().view(-1, V)
        rows = z.shape[0]
        assert targets.numel() == rows and targets.dtype == torch.int64
        tg = targets.reshape(-1).contiguous()
        loss_rows = torch.empty((rows,), dtype=torch.float32, device=z.device)
        with torch.cuda.device(z.device):
            check(lib.wkv6_softmax_xent_bf16(rows, V, _ptr(z), _ptr(tg), 1.0 / max(rows, 1), _ptr(loss_rows), _stream(z.device)))
        ctx.save_for_backward(z)          # now holds d(mean loss)/d(logits)
        ctx.shape = logits.shape
        return loss_rows.mean()

    @staticmethod
    def backward(ctx, grad_out):
        (g,) = ctx.saved_tensors
        return g.mul_(grad_out.to(g.dtype)).view(ctx.shape), None   # in place: the buffer is this function's own


def lm_loss(logits: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
    """Mean cross-entropy of bf16 ``logits`` [..., V] against int64 ``targets`` [...]; overwrites ``logits``."""
    V = logits.shape[-1]
    if logits.dtype != torch.bfloat16 or V % 8 or V > 65536 or not logits.is_contiguous():
        # same definition as the fused kernel: rows whose target lies outside [0, V) give zero loss and gradient,
        # and the mean runs over all rows
        z, t = logits.float().reshape(-1, V), targets.reshape(-1)
        valid = (t >= 0) & (t < V)
        per_row = torch.nn.functional.cross_entropy(z, t.clamp(0, V - 1), reduction="none") * valid
        return per_row.sum() / max(z.shape[0], 1)
    _check_cuda(logits, targets)
    return _LMLoss.apply(logits, targets)
