"""Fused output stage of the time-mix block: per-head GroupNorm of the WKV output, then the gate.

Mirrors ``GroupNorm`` of the reference (rwkv6_model.py:84-114: ``LayerNormalization(epsilon=64e-5)`` over the
``head_size`` channels of every head, then a ``[num_heads, head_size]`` scale and offset) and the ``x * g`` that
``TimeMix.call`` applies right after it (rwkv6_model.py:158-160), as ONE kernel per direction on the C ABI entry
points ``wkv6_groupnorm_gate_forward / _backward`` (no CPU or eager fallback).
"""
from __future__ import annotations

import ctypes

import torch

from ._lib import check, lib
from .ops import _DT, _check_cuda, _ptr, _stream

EPSILON = 64 * 1e-5  # rwkv6_model.py:85


def _rows(y: torch.Tensor, H: int, N: int) -> int:
    assert y.is_contiguous() and y.shape[-1] == H * N, "dense [..., H*N] tensors are required"
    return y.numel() // (H * N)


def groupnorm_gate_forward_raw(y, g, scale, offset, eps: float = EPSILON, gate_is_raw: bool = False):
    """``gate_is_raw``: g is the gate projection before its SiLU (rwkv6_model.py:147) and the kernel applies it."""
    _check_cuda(y, g, scale, offset)
    H, N = scale.shape
    assert g.shape == y.shape and g.dtype == y.dtype and g.is_contiguous()
    assert scale.dtype == torch.float32 and offset.dtype == torch.float32 and offset.shape == scale.shape
    out = torch.empty_like(y)
    with torch.cuda.device(y.device):
        fn = lib.wkv6_groupnorm_silu_gate_forward if gate_is_raw else lib.wkv6_groupnorm_gate_forward
        check(fn(_rows(y, H, N), H, N, _DT[y.dtype], eps, _ptr(y), _ptr(g), _ptr(scale.contiguous()),
                 _ptr(offset.contiguous()), _ptr(out), _stream(y.device)))
    return out


def groupnorm_gate_backward_raw(y, g, scale, offset, gout, eps: float = EPSILON, gate_is_raw: bool = False):
    _check_cuda(y, g, scale, offset, gout)
    H, N = scale.shape
    rows = _rows(y, H, N)
    gout = gout.contiguous()
    gy, gg = torch.empty_like(y), torch.empty_like(g)
    gscale = torch.empty((H, N), dtype=torch.float32, device=y.device)
    goffset = torch.empty((H, N), dtype=torch.float32, device=y.device)
    nbytes = lib.wkv6_groupnorm_gate_workspace_bytes(rows, H, N)
    ws = torch.empty((max(nbytes, 16),), dtype=torch.uint8, device=y.device)
    with torch.cuda.device(y.device):
        fn = lib.wkv6_groupnorm_silu_gate_backward if gate_is_raw else lib.wkv6_groupnorm_gate_backward
        check(fn(rows, H, N, _DT[y.dtype], eps, _ptr(y), _ptr(g), _ptr(scale.contiguous()),
                 _ptr(offset.contiguous()), _ptr(gout), _ptr(gy), _ptr(gg), _ptr(gscale),
                 _ptr(goffset), _ptr(ws), nbytes, _stream(y.device)))
    return gy, gg, gscale, goffset


class _GroupNormGate(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y, g, scale, offset, eps, gate_is_raw):
        ctx.save_for_backward(y, g, scale, offset)
        ctx.eps, ctx.gate_is_raw = eps, gate_is_raw
        return groupnorm_gate_forward_raw(y, g, scale, offset, eps, gate_is_raw)

    @staticmethod
    def backward(ctx, gout):
        y, g, scale, offset = ctx.saved_tensors
        gy, gg, gs, go = groupnorm_gate_backward_raw(y, g, scale, offset, gout.to(y.dtype), ctx.eps, ctx.gate_is_raw)
        return gy, gg, gs.to(scale.dtype), go.to(offset.dtype), None, None


def groupnorm_gate(y, g, scale, offset, eps: float = EPSILON, gate_is_raw: bool = False):
    """(scale * LN_head(y) + offset) * g - or * silu(g) with ``gate_is_raw`` -, differentiable in y, g, scale, offset."""
    return _GroupNormGate.apply(y.contiguous(), g.contiguous(), scale, offset, eps, gate_is_raw)


class GroupNormGate(torch.nn.Module):
    """``GroupNorm(hidden_size, head_size)`` of the reference with the gate multiplication folded in:
    ``forward(x, g) == group_norm(x) * g``."""

    def __init__(self, hidden_size: int, head_size: int, epsilon: float = EPSILON):
        super().__init__()
        assert hidden_size % head_size == 0
        self.hidden_size, self.head_size, self.num_heads, self.epsilon = hidden_size, head_size, hidden_size // head_size, epsilon
        self.scale = torch.nn.Parameter(torch.ones(self.num_heads, head_size))
        self.offset = torch.nn.Parameter(torch.zeros(self.num_heads, head_size))

    def forward(self, x, g, gate_is_raw: bool = False):
        """``gate_is_raw=True``: g is ``dense_g(xg)`` before SiLU and ``forward(x, g) == group_norm(x) * silu(g)``."""
        return groupnorm_gate(x, g, self.scale, self.offset, self.epsilon, gate_is_raw)
