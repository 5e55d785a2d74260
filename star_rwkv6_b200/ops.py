"""Torch custom ops over the C ABI (include/wkv6_b200.h).

``torch.ops.wkv6_b200.forward`` / ``backward`` take CUDA tensors, pass their device
pointers and torch's current stream to libwkv6_b200.so and return freshly allocated
outputs.  Autograd is registered on ``forward``: residuals are the five inputs plus the
checkpoint buffer the forward kernel filled, the same contract as the reference's
``RWKV_6(torch.autograd.Function)`` (rwkv_kernel/torch_rwkv_kernel.py:14-75) with the
per-batch ``gu`` summed over the batch afterwards (:73).

There is no CPU implementation: tensors that are not on a CUDA device are rejected.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch

from . import _lib
from ._lib import BF16, F16, F32, Problem, check, lib

_DT = {torch.bfloat16: BF16, torch.float16: F16, torch.float32: F32}


def out_dtype(x_dtype: torch.dtype) -> torch.dtype:
    """Output / gradient dtype policy of the reference (torch_rwkv_kernel.py:35,58): fp16 inputs give fp32."""
    return torch.float32 if x_dtype == torch.float16 else x_dtype


def _strides(t: torch.Tensor) -> Tuple[int, int]:
    """(row_stride, batch_stride) in elements of a [B,T,C] tensor whose channel dimension is contiguous."""
    B, T, C = t.shape
    assert C <= 1 or t.stride(2) == 1, "the channel dimension must be contiguous"
    ld = t.stride(1) if T > 1 else C
    bs = t.stride(0) if B > 1 else T * ld
    return ld, bs


def make_problem(r, u, head_size: int, y_dtype, variant: int, s_dtype=None, gu_dtype=torch.float32) -> Problem:
    B, T, C = r.shape
    assert C % head_size == 0
    p = Problem()
    p.B, p.T, p.H, p.N = B, T, C // head_size, head_size
    p.x_dtype = _DT[r.dtype]
    p.y_dtype = _DT[y_dtype]
    p.u_dtype = _DT[u.dtype]
    p.gu_dtype = _DT[gu_dtype]
    p.s_dtype = _DT[s_dtype] if s_dtype is not None else F32
    p.variant = variant
    p.row_stride, p.batch_stride = _strides(r)
    return p


def _out_like(ref: torch.Tensor, dtype) -> torch.Tensor:
    """Output buffer with the element layout of ``ref`` (the kernels use one stride set for inputs and outputs)."""
    if ref.is_contiguous():
        return torch.empty(ref.shape, dtype=dtype, device=ref.device)
    return torch.empty_strided(ref.shape, ref.stride(), dtype=dtype, device=ref.device)


def _same_layout(ref: torch.Tensor, *others: torch.Tensor) -> None:
    for o in others:
        assert o.shape == ref.shape and o.stride() == ref.stride(), "r, k, v, w (and gy) must share one layout"


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _stream(dev) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)


def _check_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise RuntimeError("wkv6_b200 has no CPU path: all tensors must be CUDA tensors")


def resolve_variant(r, u, head_size: int, variant: int = _lib.VARIANT_AUTO) -> int:
    p = make_problem(r, u, head_size, out_dtype(r.dtype), variant)
    rc = lib.wkv6_resolve_variant(ctypes.byref(p))
    if rc < 0:
        check(rc)
    return rc


def forward_raw(r, k, v, w, u, head_size: int, *, s_in=None, s_map=None, want_state=False, want_ckpt=False,
                variant: int = _lib.VARIANT_AUTO):
    """Launch the forward.  Returns (y, s_out or None, ckpt or None)."""
    _check_cuda(r, k, v, w, u, s_in, s_map)
    _same_layout(r, k, v, w)
    B, T, C = r.shape
    H, N = C // head_size, head_size
    ydt = out_dtype(r.dtype)
    sdt = s_in.dtype if s_in is not None else torch.float32
    p = make_problem(r, u, head_size, ydt, variant, s_dtype=sdt)
    y = _out_like(r, ydt)
    s_out = torch.empty((B, H, N, N), dtype=sdt, device=r.device) if want_state else None
    ckpt = None
    if want_ckpt:
        nbytes = lib.wkv6_ckpt_bytes(ctypes.byref(p))
        if nbytes:
            ckpt = torch.empty((nbytes,), dtype=torch.uint8, device=r.device)
    kinds = 0
    if s_in is not None:
        assert s_in.is_contiguous() and s_in.shape[1:] == (H, N, N)
        kinds = s_in.shape[0]
    if s_map is not None:
        assert s_map.dtype == torch.int64 and s_map.is_contiguous() and s_map.shape == (B,)
    if want_state and T == 0:
        # nothing to scan: the final state is the (mapped) initial state
        if s_in is None:
            s_out.zero_()
        else:
            idx = s_map if s_map is not None else (torch.zeros(B, dtype=torch.int64, device=r.device) if kinds == 1
                                                   else torch.arange(B, device=r.device))
            s_out.copy_(s_in.index_select(0, idx))
        return y, s_out, ckpt
    with torch.cuda.device(r.device):
        check(lib.wkv6_forward(ctypes.byref(p), _ptr(r), _ptr(k), _ptr(v), _ptr(w), _ptr(u), _ptr(y), _ptr(s_in),
                               _ptr(s_map), kinds, _ptr(s_out), _ptr(ckpt), _stream(r.device)))
    return y, s_out, ckpt


def backward_raw(r, k, v, w, u, gy, head_size: int, *, ckpt=None, variant: int = _lib.VARIANT_AUTO):
    """Launch the backward.  Returns (gr, gk, gv, gw, gu[B,H,N] fp32)."""
    _check_cuda(r, k, v, w, u, gy, ckpt)
    _same_layout(r, k, v, w)
    B, T, C = r.shape
    H, N = C // head_size, head_size
    ydt = out_dtype(r.dtype)
    assert gy.dtype == ydt, f"gy must have the output dtype {ydt}"
    if gy.stride() != r.stride():
        g2 = _out_like(r, ydt)
        g2.copy_(gy)
        gy = g2
    p = make_problem(r, u, head_size, ydt, variant)
    gr, gk, gv, gw = (_out_like(r, ydt) for _ in range(4))
    gu = torch.empty((B, H, N), dtype=torch.float32, device=r.device)
    nbytes = lib.wkv6_backward_workspace_bytes(ctypes.byref(p), 1 if ckpt is not None else 0)
    ws = torch.empty((nbytes,), dtype=torch.uint8, device=r.device) if nbytes else None
    with torch.cuda.device(r.device):
        check(lib.wkv6_backward(ctypes.byref(p), _ptr(r), _ptr(k), _ptr(v), _ptr(w), _ptr(u), _ptr(gy), _ptr(gr),
                                _ptr(gk), _ptr(gv), _ptr(gw), _ptr(gu), _ptr(ckpt), _ptr(ws), nbytes,
                                _stream(r.device)))
    return gr, gk, gv, gw, gu


def wkv6_decode(r, k, v, w, u, head_size: int, state=None, state_map=None, out_state=None):
    """One decode step on [B,1,C] tensors with an fp32 state [kinds,H,64,64] (None = zero).  Returns (y, new state);
    pass ``out_state=state`` for an in-place update (one state per batch row, no state_map)."""
    _check_cuda(r, k, v, w, u, state, state_map, out_state)
    B, T, C = r.shape
    assert T == 1 and head_size == 64 and r.is_contiguous()
    H = C // head_size
    ydt = out_dtype(r.dtype)
    p = make_problem(r, u, head_size, ydt, _lib.VARIANT_AUTO)
    y = torch.empty((B, 1, C), dtype=ydt, device=r.device)
    kinds = 0
    if state is not None:
        assert state.dtype == torch.float32 and state.is_contiguous() and state.shape[1:] == (H, 64, 64)
        kinds = state.shape[0]
    if out_state is None:
        out_state = torch.empty((B, H, 64, 64), dtype=torch.float32, device=r.device)
    assert out_state.dtype == torch.float32 and out_state.shape == (B, H, 64, 64) and out_state.is_contiguous()
    with torch.cuda.device(r.device):
        check(lib.wkv6_decode(ctypes.byref(p), _ptr(r), _ptr(k), _ptr(v), _ptr(w), _ptr(u), _ptr(y), _ptr(state),
                              _ptr(state_map), kinds, _ptr(out_state), _stream(r.device)))
    return y, out_state


# ---- torch.library registration -----------------------------------------------------------------

@torch.library.custom_op("wkv6_b200::forward", mutates_args=(), device_types="cuda")
def _forward_op(r: torch.Tensor, k: torch.Tensor, v: torch.Tensor, w: torch.Tensor, u: torch.Tensor,
                head_size: int, want_ckpt: bool, variant: int) -> Tuple[torch.Tensor, torch.Tensor]:
    y, _, ckpt = forward_raw(r, k, v, w, u, head_size, want_ckpt=want_ckpt, variant=variant)
    if ckpt is None:
        ckpt = torch.empty((0,), dtype=torch.uint8, device=r.device)
    return y, ckpt


@_forward_op.register_fake
def _(r, k, v, w, u, head_size, want_ckpt, variant):
    y = torch.empty(r.shape, dtype=out_dtype(r.dtype), device=r.device)
    B, T, C = r.shape
    nbytes = 0
    if want_ckpt and head_size == 64 and r.dtype == torch.bfloat16 and variant != _lib.VARIANT_SEQ and T >= 1:
        nbytes = B * (C // head_size) * ((T + 63) // 64) * 4096 * 2   # wkv6_ckpt_bytes of the chunked variant
    return y, torch.empty((nbytes,), dtype=torch.uint8, device=r.device)


@torch.library.custom_op("wkv6_b200::backward", mutates_args=(), device_types="cuda")
def _backward_op(r: torch.Tensor, k: torch.Tensor, v: torch.Tensor, w: torch.Tensor, u: torch.Tensor,
                 gy: torch.Tensor, ckpt: torch.Tensor, head_size: int, variant: int
                 ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    return backward_raw(r, k, v, w, u, gy, head_size, ckpt=ckpt if ckpt.numel() else None, variant=variant)


@_backward_op.register_fake
def _(r, k, v, w, u, gy, ckpt, head_size, variant):
    B, T, C = r.shape
    g = [torch.empty(r.shape, dtype=out_dtype(r.dtype), device=r.device) for _ in range(4)]
    return (*g, torch.empty((B, C // head_size, head_size), dtype=torch.float32, device=r.device))


def _setup_context(ctx, inputs, output):
    r, k, v, w, u, head_size, want_ckpt, variant = inputs
    _, ckpt = output
    ctx.save_for_backward(r, k, v, w, u, ckpt)
    ctx.head_size = head_size
    ctx.variant = variant


def _autograd_backward(ctx, gy, _g_ckpt):
    r, k, v, w, u, ckpt = ctx.saved_tensors
    gr, gk, gv, gw, gu_b = torch.ops.wkv6_b200.backward(r, k, v, w, u, gy, ckpt, ctx.head_size, ctx.variant)
    gu = gu_b.sum(0).to(u.dtype).reshape(u.shape)
    xdt = r.dtype
    return gr.to(xdt), gk.to(xdt), gv.to(xdt), gw.to(xdt), gu, None, None, None


_forward_op.register_autograd(_autograd_backward, setup_context=_setup_context)


def wkv6(r, k, v, w, u, head_size: int, variant: int = _lib.VARIANT_AUTO) -> torch.Tensor:
    """Differentiable WKV6 with a zero initial state: y[B,T,C] from r,k,v,w [B,T,C] and u [H,N]."""
    need_grad = torch.is_grad_enabled() and any(t.requires_grad for t in (r, k, v, w, u))
    y, _ = torch.ops.wkv6_b200.forward(r, k, v, w, u, head_size, need_grad, variant)
    return y


def wkv6_with_state(r, k, v, w, u, head_size: int, init_state=None, state_map=None,
                    variant: int = _lib.VARIANT_AUTO):
    """Forward only, with an optional initial state and the final state returned (no autograd), as the
    reference's with-state kernel (rwkv_kernel/jax_kernel/rwkv_kernels.cu:165-190)."""
    with torch.no_grad():
        y, s_out, _ = forward_raw(r, k, v, w, u, head_size, s_in=init_state, s_map=state_map, want_state=True,
                                  variant=variant)
    return y, s_out
