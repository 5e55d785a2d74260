"""Fused element-wise stages of a decode step (one token per sequence) around the matrix products of an RWKV-6 block:
thin wrappers over the C ABI (``wkv6_decode_ln_shift_mix``, ``wkv6_decode_lora_mix``, ``wkv6_decode_relu_sq``,
``wkv6_decode_sigmoid_mul_add``, ``wkv6_decode_gated``).  At T = 1 every tensor is [B, D]; these stages cost launch
latency only, so a layer's ~30 framework operations become 8 launches besides its matrix products.
Expressions: rwkv6_model.py:37-44, 128-160 (time mix) and :48-83 (channel mix) for a single token.
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib
from ._lib import check, lib
from .ops import _check_cuda, _DT, _ptr, _stream, make_problem, out_dtype

_MIX_PERM_RKVGW = (ctypes.c_int32 * 5)(0, 1, 2, 4, 3)   # mixes arrive in the order r, k, v, w, g; store them as r, k, v, g, w


def ln_shift_mix(x, ln_weight, ln_bias, eps, prev, mu0, mu1=None, want_xa_xs=False):
    """x, prev: [B, D] (prev is replaced by LayerNorm(x)).  Returns (mix0, mix1 or None, xa or None, xs or None)."""
    _check_cuda(x, ln_weight, ln_bias, prev, mu0, mu1)
    B, D = x.shape
    assert x.is_contiguous() and prev.is_contiguous() and prev.shape == x.shape and prev.dtype == x.dtype
    assert ln_weight.dtype == x.dtype and ln_bias.dtype == x.dtype and mu0.dtype == torch.float32
    mix0 = torch.empty_like(x)
    mix1 = torch.empty_like(x) if mu1 is not None else None
    xa = torch.empty_like(x) if want_xa_xs else None
    xs = torch.empty_like(x) if want_xa_xs else None
    with torch.cuda.device(x.device):
        check(lib.wkv6_decode_ln_shift_mix(B, D, _DT[x.dtype], float(eps), _ptr(x), _ptr(ln_weight), _ptr(ln_bias), _ptr(prev),
                                           _ptr(mu0), _ptr(mu1), _ptr(xa), _ptr(xs), _ptr(mix0), _ptr(mix1), _stream(x.device)))
    return mix0, mix1, xa, xs


def lora_mix(h, dense_b, bias_b, xa, xs):
    """h [B, 5R] (before tanh), dense_b [5, R, D], bias_b [5, 1, D] in the order r, k, v, w, g.
    Returns [5, B, D] in the order r, k, v, g, w (the four inputs of the big projections first)."""
    _check_cuda(h, dense_b, bias_b, xa, xs)
    B, D = xa.shape
    R = dense_b.shape[1]
    assert h.shape == (B, 5 * R) and dense_b.shape == (5, R, D) and bias_b.numel() == 5 * D
    assert all(t.is_contiguous() and t.dtype == xa.dtype for t in (h, dense_b, bias_b, xa, xs))
    out = torch.empty((5, B, D), dtype=xa.dtype, device=xa.device)
    with torch.cuda.device(xa.device):
        check(lib.wkv6_decode_lora_mix(B, D, R, _DT[xa.dtype], _ptr(h), _ptr(dense_b), _ptr(bias_b), _ptr(xa), _ptr(xs),
                                       _ptr(out), _MIX_PERM_RKVGW, _stream(xa.device)))
    return out


def relu_sq(x):
    _check_cuda(x)
    assert x.is_contiguous()
    out = torch.empty_like(x)
    with torch.cuda.device(x.device):
        check(lib.wkv6_decode_relu_sq(x.numel(), _DT[x.dtype], _ptr(x), _ptr(out), _stream(x.device)))
    return out


def sigmoid_mul_add(x, r, kv):
    """x + sigmoid(r) * kv."""
    _check_cuda(x, r, kv)
    assert x.is_contiguous() and r.is_contiguous() and kv.is_contiguous() and x.shape == r.shape == kv.shape
    assert x.dtype == r.dtype == kv.dtype
    out = torch.empty_like(x)
    with torch.cuda.device(x.device):
        check(lib.wkv6_decode_sigmoid_mul_add(x.numel(), _DT[x.dtype], _ptr(x), _ptr(r), _ptr(kv), _ptr(out), _stream(x.device)))
    return out


def wkv6_decode_gated(r, k, v, w, u, g_raw, gn_scale, gn_offset, eps, head_size: int, state):
    """One decode step on [B,1,C] (or [B,C]) tensors with the fp32 state [B,H,64,64] updated in place, followed by the
    per-head GroupNorm and the SiLU gate: returns (GroupNorm(y) * scale + offset) * silu(g_raw)."""
    _check_cuda(r, k, v, w, u, g_raw, gn_scale, gn_offset, state)
    B, C = r.shape[0], r.shape[-1]
    assert head_size == 64 and r.numel() == B * C and all(t.is_contiguous() for t in (r, k, v, w, g_raw))
    H = C // head_size
    assert state.dtype == torch.float32 and state.shape == (B, H, 64, 64) and state.is_contiguous()
    assert gn_scale.dtype == gn_offset.dtype == torch.float32 and gn_scale.numel() == C
    ydt = out_dtype(r.dtype)
    p = make_problem(r.view(B, 1, C), u, head_size, ydt, _lib.VARIANT_AUTO)
    out = torch.empty(r.shape, dtype=ydt, device=r.device)
    with torch.cuda.device(r.device):
        check(lib.wkv6_decode_gated(ctypes.byref(p), _ptr(r), _ptr(k), _ptr(v), _ptr(w), _ptr(u), _ptr(g_raw), _ptr(gn_scale),
                                    _ptr(gn_offset), float(eps), _ptr(out), _ptr(state), None, B, _ptr(state),
                                    _stream(r.device)))
    return out
