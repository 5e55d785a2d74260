"""Input stage of the time-mix block: from the block input x to the five tensors that feed the r, k, v, w, g
projections (TimeMix.call, rwkv6_model.py:128-146):

    x_shift = shift(x) - x                              (TimeShift, rwkv6_model.py:37-44)
    x_mix   = x + x_shift * time_mix_x
    l_i     = tanh(x_mix A_i) B_i + b_i                 (DecomposerDense, rwkv6_model.py:11-24), i in r, k, v, w, g
    x_i     = x + x_shift * l_i

The two interpolation steps are the fused kernels behind ``wkv6_shift_mix_forward / _backward`` (x is read once, no
shifted copy is materialised); the two small matrix products are plain library GEMMs (torch.matmul / baddbmm).
"""
from __future__ import annotations

import ctypes

import torch

from ._lib import check, lib
from .ops import _DT, _check_cuda, _ptr, _stream


def _shift_mix_fwd(x, m, vector: bool):
    B, T, C = x.shape
    nmix = 1 if vector else m.shape[0]
    out = torch.empty((B, T, C) if vector else (nmix, B, T, C), dtype=x.dtype, device=x.device)
    with torch.cuda.device(x.device):
        check(lib.wkv6_shift_mix_forward(B, T, C, _DT[x.dtype], nmix, 1 if vector else 0, _ptr(x), _ptr(m), _ptr(out),
                                         _stream(x.device)))
    return out


def _shift_mix_bwd(x, m, gout, vector: bool):
    B, T, C = x.shape
    nmix = 1 if vector else m.shape[0]
    gx = torch.empty_like(x)
    gm = torch.empty((C,), dtype=torch.float32, device=x.device) if vector else torch.empty_like(m)
    nbytes = lib.wkv6_shift_mix_workspace_bytes(B, T, C, 1 if vector else 0)
    ws = torch.empty((nbytes,), dtype=torch.uint8, device=x.device) if nbytes else None
    with torch.cuda.device(x.device):
        check(lib.wkv6_shift_mix_backward(B, T, C, _DT[x.dtype], nmix, 1 if vector else 0, _ptr(x), _ptr(m), _ptr(gout),
                                          _ptr(gx), _ptr(gm), _ptr(ws), nbytes, _stream(x.device)))
    return gx, gm


class _ShiftMixVec(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, mu):
        _check_cuda(x, mu)
        x = x.contiguous()
        mu32 = mu.detach().to(torch.float32).contiguous()
        ctx.save_for_backward(x, mu32)
        ctx.mu_dtype = mu.dtype
        return _shift_mix_fwd(x, mu32, True)

    @staticmethod
    def backward(ctx, gout):
        x, mu32 = ctx.saved_tensors
        gx, gmu = _shift_mix_bwd(x, mu32, gout.to(x.dtype).contiguous(), True)
        return gx, gmu.to(ctx.mu_dtype)


class _ShiftMixTensors(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, m):
        _check_cuda(x, m)
        x, m = x.contiguous(), m.contiguous()
        assert m.dtype == x.dtype and m.shape[1:] == x.shape and m.shape[0] in (1, 5)
        ctx.save_for_backward(x, m)
        return _shift_mix_fwd(x, m, False)

    @staticmethod
    def backward(ctx, gout):
        x, m = ctx.saved_tensors
        return _shift_mix_bwd(x, m, gout.to(x.dtype).contiguous(), False)


def shift_mix_vector(x, mu):
    """x + (shift(x) - x) * mu for x [B,T,C] and one mixing vector mu [C]."""
    return _ShiftMixVec.apply(x, mu)


def shift_mix_tensors(x, m):
    """x + (shift(x) - x) * m[j] for x [B,T,C] and m [nmix,B,T,C] (nmix = 1 or 5); returns [nmix,B,T,C]."""
    return _ShiftMixTensors.apply(x, m)


class TimeMixInputs(torch.nn.Module):
    """The five mixed inputs (xr, xk, xv, xw, xg) of the reference's TimeMix from the block input."""

    ORDER = ("r", "k", "v", "w", "g")

    def __init__(self, hidden_size: int, decomposer_size: int = 32):
        super().__init__()
        D, R = hidden_size, decomposer_size
        self.hidden_size, self.decomposer_size = D, R
        self.time_mix_x = torch.nn.Parameter(torch.zeros(D))
        self.dense_a = torch.nn.Parameter(torch.randn(D, 5 * R) * D ** -0.5)   # dense_a of the five DecomposerDense, side by side
        self.dense_b = torch.nn.Parameter(torch.randn(5, R, D) * R ** -0.5)    # dense_b kernels
        self.bias_b = torch.nn.Parameter(torch.zeros(5, 1, D))                 # dense_b biases (use_bias=True)

    def forward(self, x):
        B, T, D = x.shape
        x_mix = shift_mix_vector(x, self.time_mix_x)
        h = torch.tanh(x_mix.reshape(B * T, D) @ self.dense_a.to(x.dtype))                      # [B*T, 5R]
        h = h.reshape(B * T, 5, self.decomposer_size).transpose(0, 1)                            # [5, B*T, R]
        l = torch.baddbmm(self.bias_b.to(x.dtype), h, self.dense_b.to(x.dtype))                  # [5, B*T, D]
        return shift_mix_tensors(x, l.reshape(5, B, T, D))                                       # xr, xk, xv, xw, xg
