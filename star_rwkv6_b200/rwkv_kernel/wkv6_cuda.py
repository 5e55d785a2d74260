"""Drop-in for the module the reference builds with ``torch.utils.cpp_extension.load(name="wkv6", ...)``
(rwkv_kernel/torch_rwkv_kernel.py:11-13): the nine functions of rwkv_kernel/torch_kernel/wkv6_op.cpp:22-60 with the
same names, argument orders and out-parameter convention (every output tensor is allocated by the caller), served by
the B200 library through its C ABI.  In the reference's operator, replacing the ``load(...)`` call by

    from star_rwkv6_b200.rwkv_kernel import wkv6_cuda

leaves its ``RWKV_6`` autograd function (torch_rwkv_kernel.py:14-75) working unchanged.

    forward_{fp32,bf16,fp16}(B, T, C, H, r, k, v, w, u, y)
    backward_{fp32,bf16,fp16}(B, T, C, H, r, k, v, w, u, gy, gr, gk, gv, gw, gu)        gu: [B, C], one row per batch row
    forward_with_state_{fp32,bf16,fp16}(B, T, C, H, S, map, r, k, v, w, u, s, y, ys)     S: whether s / map are given

Dtype policy as in the reference (torch_rwkv_kernel.py:35, 58): fp16 inputs give fp32 outputs.  States (s, ys) are
``[kinds or B, H, N, N]`` in the layout ``S[b, h, key, value]``, fp32 or bf16.  T has no compile-time cap and the head
size is C // H (8, 16, 32 or 64) instead of the ``-D_N_`` build flag.  The kernels run on torch's current stream.
"""
from __future__ import annotations

import ctypes

import torch

from .. import _lib
from .._lib import check, lib
from ..ops import _DT, _ptr, _stream, make_problem, out_dtype

_NAMES = {"fp32": torch.float32, "bf16": torch.bfloat16, "fp16": torch.float16}


def _check(dtype, B, T, C, H, *tensors):
    assert C % H == 0
    for t in tensors:
        assert t.is_cuda and t.is_contiguous(), "tensors must be contiguous CUDA tensors"
    for t in tensors[:4]:
        assert t.dtype == dtype and tuple(t.shape) == (B, T, C), "r, k, v, w must be [B, T, C] of the function's dtype"


def _forward(dtype, B, T, C, H, r, k, v, w, u, y, s=None, s_map=None, ys=None):
    _check(dtype, B, T, C, H, r, k, v, w, u, y)
    ydt = out_dtype(dtype)
    assert y.dtype == ydt and tuple(y.shape) == (B, T, C)
    sdt = ys.dtype if ys is not None else torch.float32
    if s is not None:
        assert s.dtype == sdt and s.is_contiguous() and tuple(s.shape[1:]) == (H, C // H, C // H)
        assert s_map is not None and s_map.dtype == torch.int64 and tuple(s_map.shape) == (B,) and s_map.is_contiguous()
    p = make_problem(r, u.reshape(H, C // H), C // H, ydt, _lib.VARIANT_AUTO, s_dtype=sdt)
    with torch.cuda.device(r.device):
        check(lib.wkv6_forward(ctypes.byref(p), _ptr(r), _ptr(k), _ptr(v), _ptr(w), _ptr(u), _ptr(y), _ptr(s),
                               _ptr(s_map) if s is not None else None, s.shape[0] if s is not None else 0, _ptr(ys), None,
                               _stream(r.device)))


def _backward(dtype, B, T, C, H, r, k, v, w, u, gy, gr, gk, gv, gw, gu):
    _check(dtype, B, T, C, H, r, k, v, w, u, gy, gr, gk, gv, gw, gu)
    ydt = out_dtype(dtype)
    for t in (gy, gr, gk, gv, gw):
        assert t.dtype == ydt and tuple(t.shape) == (B, T, C)
    assert gu.dtype in (ydt, torch.float32) and gu.numel() == B * C
    p = make_problem(r, u.reshape(H, C // H), C // H, ydt, _lib.VARIANT_AUTO, gu_dtype=gu.dtype)
    nbytes = lib.wkv6_backward_workspace_bytes(ctypes.byref(p), 0)
    ws = torch.empty((nbytes,), dtype=torch.uint8, device=r.device) if nbytes else None
    with torch.cuda.device(r.device):
        check(lib.wkv6_backward(ctypes.byref(p), _ptr(r), _ptr(k), _ptr(v), _ptr(w), _ptr(u), _ptr(gy), _ptr(gr), _ptr(gk),
                                _ptr(gv), _ptr(gw), _ptr(gu), None, _ptr(ws), nbytes, _stream(r.device)))


def _forward_with_state(dtype, B, T, C, H, S, s_map, r, k, v, w, u, s, y, ys):
    assert ys is not None and ys.is_cuda and ys.is_contiguous() and tuple(ys.shape) == (B, H, C // H, C // H)
    assert ys.dtype in (torch.float32, torch.bfloat16), "states are fp32 or bf16"
    if not S:
        s, s_map = None, None
    _forward(dtype, B, T, C, H, r, k, v, w, u, y, s=s, s_map=s_map, ys=ys)


def _bind(kind, fn, name, dtype):
    def call(*args):
        return fn(dtype, *args)
    call.__name__ = f"{kind}_{name}"
    call.__doc__ = f"wkv6 {kind.replace('_', ' ')} {name} (rwkv_kernel/torch_kernel/wkv6_op.cpp)"
    return call


for _name, _dtype in _NAMES.items():
    globals()[f"forward_{_name}"] = _bind("forward", _forward, _name, _dtype)
    globals()[f"backward_{_name}"] = _bind("backward", _backward, _name, _dtype)
    globals()[f"forward_with_state_{_name}"] = _bind("forward_with_state", _forward_with_state, _name, _dtype)

__all__ = [f"{k}_{n}" for k in ("forward", "backward", "forward_with_state") for n in _NAMES]
