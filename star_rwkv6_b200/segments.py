"""WKV6 with the sequence split along T: inside one GPU (more independent work when there are few (batch, head)
pairs) and across GPUs (each rank holds a contiguous T range; the N x N per-head states are carried rank to rank).

A segment is summarised as an affine map of the state, S -> 2^dec * S + b (dec per key channel, b = the state the
segment builds from zero).  Maps compose associatively, so every rank gathers all summaries (H*(N*N+N)*4 bytes per
segment), runs the same exclusive scan and starts its segments from the right states; the backward does the mirror
image for the reverse state.  The reference has no counterpart: its kernels cap T at a compile-time constant
(rwkv_kernel/jax_kernel/rwkv_kernels.cu:351) and its only long-sequence mechanism is forward state chaining
(rwkv_kernel/__init__.py:14-37).

The numerical work is done by a *backend* (the CUDA library by default); the orchestration - reshaping, gathering,
scanning, slicing - is backend-independent so that it can be exercised on CPU ranks with the oracle as backend.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch
import torch.distributed as dist


class LibraryBackend:
    """Chunked sm_100a kernels through the C ABI (bf16 r,k,v,w,gy; N = 64).

    ``reuse_buffers=True`` keeps every output, summary, checkpoint and workspace buffer of the first call and hands the
    same memory out again on later calls of the same shapes, so that a step allocates nothing (a training loop that
    consumes the results of one step before it starts the next; results of an earlier call are overwritten)."""

    def __init__(self, head_size: int, reuse_buffers: bool = False):
        from . import _lib, ops
        self.L, self.ops, self.N = _lib, ops, head_size
        self.reuse = reuse_buffers
        self._bufs = {}
        self.scan_only_summaries = True   # summary() accepts scan_only_segments

    def _buf(self, name, shape, dtype, device):
        if not self.reuse:
            return torch.empty(shape, dtype=dtype, device=device)
        key = (name, tuple(shape), dtype, str(device))
        t = self._bufs.get(key)
        if t is None:
            t = self._bufs[key] = torch.empty(shape, dtype=dtype, device=device)
        return t

    def _problem(self, x, u=None):
        u = u if u is not None else torch.empty(0, dtype=torch.float32, device=x.device)
        return self.ops.make_problem(x, u, self.N, x.dtype, self.L.VARIANT_CHUNK)

    def _stream(self, x):
        return ctypes.c_void_p(torch.cuda.current_stream(x.device).cuda_stream)

    def summary(self, x1, x2, w, reverse: bool, scan_only_segments: int = 0):
        """Summaries of the rows of [B*G, Tseg, C] tensors.  ``scan_only_segments`` = G > 0: leave out the one segment per
        sequence that an exclusive scan never reads (see wkv6_segment_summary_for_scan); its rows come back unwritten."""
        Bn, T, C = x1.shape
        H = C // self.N
        tag = "rev" if reverse else "fwd"
        state = self._buf("sum_state_" + tag, (Bn, H, self.N, self.N), torch.float32, x1.device)
        dec = self._buf("sum_dec_" + tag, (Bn, H, self.N), torch.float32, x1.device)
        p = self._problem(x1)
        ptr = self.ops._ptr
        with torch.cuda.device(x1.device):
            if scan_only_segments > 0:
                self.L.check(self.L.lib.wkv6_segment_summary_for_scan(ctypes.byref(p), ptr(x1), ptr(x2), ptr(w), int(reverse),
                                                                      scan_only_segments, ptr(state), ptr(dec), self._stream(x1)))
            else:
                self.L.check(self.L.lib.wkv6_segment_summary(ctypes.byref(p), ptr(x1), ptr(x2), ptr(w), int(reverse), ptr(state),
                                                             ptr(dec), self._stream(x1)))
        return state, dec

    def scan(self, B, H, G, dec, state, s0, reverse: bool):
        tag = "rev" if reverse else "fwd"
        out = self._buf("scan_out_" + tag, tuple(state.shape), torch.float32, state.device)
        last = self._buf("scan_last_" + tag, (B, H, self.N, self.N), torch.float32, state.device)
        ptr = self.ops._ptr
        with torch.cuda.device(state.device):
            self.L.check(self.L.lib.wkv6_state_scan(B, H, self.N, G, ptr(dec), ptr(state), ptr(s0), ptr(out), ptr(last),
                                                    int(reverse), self._stream(state)))
        return out, last

    def forward(self, r, k, v, w, u, s_in, want_ckpt: bool):
        if not self.reuse:
            y, _, ckpt = self.ops.forward_raw(r, k, v, w, u, self.N, s_in=s_in, want_ckpt=want_ckpt, variant=self.L.VARIANT_CHUNK)
            return y, ckpt
        Bn, T, C = r.shape
        p = self.ops.make_problem(r, u, self.N, r.dtype, self.L.VARIANT_CHUNK)
        y = self._buf("y", (Bn, T, C), r.dtype, r.device)
        nbytes = self.L.lib.wkv6_ckpt_bytes(ctypes.byref(p)) if want_ckpt else 0
        ckpt = self._buf("ckpt", (nbytes,), torch.uint8, r.device) if nbytes else None
        ptr = self.ops._ptr
        with torch.cuda.device(r.device):
            self.L.check(self.L.lib.wkv6_forward(ctypes.byref(p), ptr(r), ptr(k), ptr(v), ptr(w), ptr(u), ptr(y), ptr(s_in), None,
                                                 s_in.shape[0] if s_in is not None else 0, None, ptr(ckpt), self._stream(r)))
        return y, ckpt

    def backward(self, r, k, v, w, u, gy, ckpt, ab_in):
        Bn, T, C = r.shape
        H = C // self.N
        p = self.ops.make_problem(r, u, self.N, r.dtype, self.L.VARIANT_CHUNK)
        g = [self._buf("g" + n, (Bn, T, C), r.dtype, r.device) for n in "rkvw"]
        gu = self._buf("gu", (Bn, H, self.N), torch.float32, r.device)
        ptr = self.ops._ptr
        nbytes = self.L.lib.wkv6_backward_workspace_bytes(ctypes.byref(p), 1)
        ws = self._buf("ws", (nbytes,), torch.uint8, r.device) if nbytes else None
        with torch.cuda.device(r.device):
            self.L.check(self.L.lib.wkv6_backward_seeded(ctypes.byref(p), ptr(r), ptr(k), ptr(v), ptr(w), ptr(u), ptr(gy),
                                                         *(ptr(x) for x in g), ptr(gu), ptr(ckpt), ptr(ab_in), ptr(ws),
                                                         nbytes, self._stream(r)))
        return (*g, gu)


    def sum_rows(self, rows: torch.Tensor) -> torch.Tensor:
        """[R, H, N] fp32 -> [H, N]: the per-segment gu rows added up (one small launch)."""
        rows = rows.contiguous()
        out = self._buf("gu_sum", tuple(rows.shape[1:]), torch.float32, rows.device)
        n = out.numel()
        with torch.cuda.device(rows.device):
            self.L.check(self.L.lib.wkv6_sum_rows(self.ops._ptr(rows), rows.shape[0], n, self.ops._ptr(out), self._stream(rows)))
        return out


def auto_segments(B: int, T: int, H: int, target_sequences: int = 256, max_segments: int = 16, min_tokens: int = 256) -> int:
    """Number of segments that brings B*H*G independent sequences to about two per SM (the kernels run two CTAs per
    SM, one CTA per sequence): a power of two, dividing T, with at least ``min_tokens`` tokens per segment."""
    G = 1
    while (B * H * G < target_sequences and G < max_segments and T % (2 * G) == 0 and T // (2 * G) >= min_tokens):
        G *= 2
    return G


def _split(x: torch.Tensor, G: int) -> torch.Tensor:
    """[B, T, C] -> [B*G, T/G, C] (a view: segment g of batch row b becomes row b*G + g)."""
    B, T, C = x.shape
    assert T % G == 0, "T must be a multiple of the number of segments"
    assert x.is_contiguous()
    return x.view(B * G, T // G, C)


def _gather_segments(x: torch.Tensor, B: int, G: int, group) -> torch.Tensor:
    """Summaries [B*G, ...] of every rank -> [B*(R*G), ...] with the segments of rank 0 first along g."""
    if group is None or dist.get_world_size(group) == 1:
        return x
    R = dist.get_world_size(group)
    parts = [torch.empty_like(x) for _ in range(R)]
    dist.all_gather(parts, x.contiguous(), group=group)
    allx = torch.stack(parts, 0).view(R, B, G, *x.shape[1:])          # [R, B, G, ...]
    return allx.transpose(0, 1).reshape(B * R * G, *x.shape[1:])       # [B, R, G, ...] -> [B*R*G, ...]


def _local_segments(x: torch.Tensor, B: int, G: int, group) -> torch.Tensor:
    if group is None or dist.get_world_size(group) == 1:
        return x
    R, rank = dist.get_world_size(group), dist.get_rank(group)
    return x.view(B, R, G, *x.shape[1:])[:, rank].reshape(B * G, *x.shape[1:]).contiguous()


def segmented_forward(backend, r, k, v, w, u, segments: int, init_state: Optional[torch.Tensor] = None,
                      want_ckpt: bool = False, group=None, need_last: bool = True):
    """Forward over local tensors [B, T_local, C].  Returns (y, state after the whole sequence, context for backward).

    ``need_last=False`` (one rank only): the caller does not want the final state, so the summary of every sequence's last
    segment - and, in the backward, of its first - is not computed (None comes back in place of the state)."""
    B, T, C = r.shape
    G = segments
    rs, ks, vs, ws = (_split(x, G) for x in (r, k, v, w))
    R = 1 if group is None else dist.get_world_size(group)
    lean = (not need_last) and R == 1 and getattr(backend, "scan_only_summaries", False)
    state, dec = backend.summary(ks, vs, ws, False, G) if lean else backend.summary(ks, vs, ws, False)
    H = state.shape[1]
    state_all, dec_all = _gather_segments(state, B, G, group), _gather_segments(dec, B, G, group)
    s_in_all, last = backend.scan(B, H, R * G, dec_all, state_all, init_state, False)
    s_in = _local_segments(s_in_all, B, G, group)
    y, ckpt = backend.forward(rs, ks, vs, ws, u, s_in, want_ckpt)
    ctx = dict(dec_all=dec_all, ckpt=ckpt, B=B, G=G, H=H, group=group, lean=lean)
    return y.view(B, T, C), (None if lean else last), ctx


def segmented_backward(backend, ctx, r, k, v, w, u, gy):
    """Gradients for local tensors [B, T_local, C]; gu is summed over batch rows, segments and ranks."""
    B, G, H, group = ctx["B"], ctx["G"], ctx["H"], ctx["group"]
    T, C = r.shape[1], r.shape[2]
    rs, ks, vs, ws, gs = (_split(x, G) for x in (r, k, v, w, gy))
    R = 1 if group is None else dist.get_world_size(group)
    if ctx.get("lean"):  # the reverse summaries bring the decays their scan needs (the forward left out the last segment's)
        astate, dec_all = backend.summary(rs, gs, ws, True, G)
    else:
        astate, _ = backend.summary(rs, gs, ws, True)
        dec_all = ctx["dec_all"]
    astate_all = _gather_segments(astate, B, G, group)
    a_in_all, _ = backend.scan(B, H, R * G, dec_all, astate_all, None, True)
    a_in = _local_segments(a_in_all, B, G, group)
    gr, gk, gv, gw, gu_rows = backend.backward(rs, ks, vs, ws, u, gs, ctx["ckpt"], a_in)
    gu = backend.sum_rows(gu_rows) if hasattr(backend, "sum_rows") else gu_rows.sum(0)
    if R > 1:
        dist.all_reduce(gu, op=dist.ReduceOp.SUM, group=group)
    return gr.view(B, T, C), gk.view(B, T, C), gv.view(B, T, C), gw.view(B, T, C), gu


class _SegmentedWKV6(torch.autograd.Function):
    @staticmethod
    def forward(ctx, r, k, v, w, u, backend, segments, group):
        y, _, c = segmented_forward(backend, r, k, v, w, u, segments, want_ckpt=True, group=group, need_last=False)
        ctx.save_for_backward(r, k, v, w, u)
        ctx.c, ctx.backend = c, backend
        return y

    @staticmethod
    def backward(ctx, gy):
        r, k, v, w, u = ctx.saved_tensors
        gr, gk, gv, gw, gu = segmented_backward(ctx.backend, ctx.c, r, k, v, w, u, gy.contiguous())
        return gr, gk, gv, gw, gu.to(u.dtype).reshape(u.shape), None, None, None


def wkv6_segmented(r, k, v, w, u, head_size: int, segments: int, group=None, backend=None):
    """Differentiable WKV6 (zero initial state) with every local sequence cut into ``segments`` pieces; with
    ``group`` the T axis is additionally sharded over the ranks of the group in rank order."""
    backend = backend or LibraryBackend(head_size)
    return _SegmentedWKV6.apply(r, k, v, w, u, backend, segments, group)
