"""Differentiable activations of the channel-mix block on the library's kernels (C ABI ``wkv6_relu_sq_*`` /
``wkv6_sigmoid_mul_*``): ``relu_sq(x) = max(x, 0)^2`` and ``sigmoid_mul(r, kv) = sigmoid(r) * kv``, the expressions of
the reference's ChannelMix (rwkv6_model.py:47-48, :64, :83), each as one kernel per direction instead of the two to
three framework kernels with an HBM round trip each.  CUDA tensors only; any shape, dense."""
from __future__ import annotations

import torch

from ._lib import check, lib
from .ops import _DT, _check_cuda, _ptr, _stream


def _dense(t: torch.Tensor) -> torch.Tensor:
    return t if t.is_contiguous() else t.contiguous()


class _ReluSq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        _check_cuda(x)
        x = _dense(x)
        out = torch.empty_like(x)
        with torch.cuda.device(x.device):
            check(lib.wkv6_relu_sq_forward(x.numel(), _DT[x.dtype], _ptr(x), _ptr(out), _stream(x.device)))
        ctx.save_for_backward(x)
        return out

    @staticmethod
    def backward(ctx, gout):
        (x,) = ctx.saved_tensors
        gout = _dense(gout)
        gx = torch.empty_like(x)
        with torch.cuda.device(x.device):
            check(lib.wkv6_relu_sq_backward(x.numel(), _DT[x.dtype], _ptr(x), _ptr(gout), _ptr(gx), _stream(x.device)))
        return gx


class _SigmoidMul(torch.autograd.Function):
    @staticmethod
    def forward(ctx, r, kv):
        _check_cuda(r, kv)
        assert r.shape == kv.shape and r.dtype == kv.dtype
        r, kv = _dense(r), _dense(kv)
        out = torch.empty_like(r)
        with torch.cuda.device(r.device):
            check(lib.wkv6_sigmoid_mul_forward(r.numel(), _DT[r.dtype], _ptr(r), _ptr(kv), _ptr(out), _stream(r.device)))
        ctx.save_for_backward(r, kv)
        return out

    @staticmethod
    def backward(ctx, gout):
        r, kv = ctx.saved_tensors
        gout = _dense(gout)
        gr, gkv = torch.empty_like(r), torch.empty_like(kv)
        with torch.cuda.device(r.device):
            check(lib.wkv6_sigmoid_mul_backward(r.numel(), _DT[r.dtype], _ptr(r), _ptr(kv), _ptr(gout), _ptr(gr), _ptr(gkv),
                                                _stream(r.device)))
        return gr, gkv


def relu_sq(x: torch.Tensor) -> torch.Tensor:
    """max(x, 0)^2 (the activation of the reference's dense_key)."""
    return _ReluSq.apply(x)


def sigmoid_mul(r: torch.Tensor, kv: torch.Tensor) -> torch.Tensor:
    """sigmoid(r) * kv (the receptance gate of the reference's ChannelMix)."""
    return _SigmoidMul.apply(r, kv)
