"""WKV6 forward + backward for tensors that live in (pinned) host memory.

The reference operator takes device tensors; a caller whose activations sit in host memory pays two PCIe transfers
per call (5 tensors in, 5 out), which dwarf the kernels.  ``HostPipeline`` streams the batch rows through the GPU in
slices on a few CUDA streams, so that the host-to-device copy of one slice, the kernels of the previous one and the
device-to-host copy of the one before run at the same time (the two copy directions use separate DMA engines); a call
then costs about one direction of PCIe traffic instead of both plus the kernels.  Rows are independent (the recurrence
never crosses a batch row) and so are heads, so slicing changes no result; the first and the last row are cut into
two head groups to shorten the fill and the drain of the pipeline.  Every slot owns its device buffers, allocated once: the
calls themselves go straight to the C ABI and allocate nothing.
"""
from __future__ import annotations

import collections
import ctypes
from typing import Dict, Optional

import torch

from . import _lib
from ._lib import check, lib
from .ops import _ptr, _stream, make_problem, out_dtype

_IN = ("r", "k", "v", "w", "gy")
_OUT = ("y", "gr", "gk", "gv", "gw")


class HostPipeline:
    def __init__(self, T: int, H: int, head_size: int, dtype=torch.bfloat16, device=None, rows_per_slice: int = 1,
                 slots: int = 6, variant: int = _lib.VARIANT_AUTO, ramp: bool = True):
        """``ramp`` (an attribute, may be changed between calls): cut the first and the last batch row into two head groups
        (heads are as independent as rows), so that the first kernels start and the last copy back ends half a row's transfer
        earlier - for one call at a time; a loop that keeps two calls in flight (``submit`` / ``wait``) is faster without it
        (14.7 against 15.3 ms per call at the same shape: the next call's fill covers the drain, and whole rows are plain copies).  Measured at B8 T4096
        H32 with six slots: 17.0 ms per call against 17.4 ms without (same GPU, alternating runs); finer groups (eighths) were slower, their pitched copies being short."""
        self.device = torch.device(device if device is not None else "cuda")
        self.T, self.H, self.N, self.rows, self.variant = T, H, head_size, rows_per_slice, variant
        self.ramp = bool(ramp) and rows_per_slice == 1 and H % 2 == 0
        C = H * head_size
        ydt = out_dtype(dtype)
        self.slots = []
        with torch.cuda.device(self.device):
            for _ in range(max(1, slots)):
                s = {n: torch.empty((rows_per_slice, T, C), dtype=dtype if n != "gy" else ydt, device=self.device) for n in _IN}
                s.update({n: torch.empty((rows_per_slice, T, C), dtype=ydt, device=self.device) for n in _OUT})
                s["gu"] = torch.empty((rows_per_slice, H, head_size), dtype=torch.float32, device=self.device)
                s["stream"] = torch.cuda.Stream(self.device)
                self.slots.append(s)
            # two copies of u and a stream of their own for its upload, so that a call submitted while the one before is
            # still running neither overwrites the u that call reads nor waits for it
            self.u2 = [torch.empty((H, head_size), dtype=torch.float32, device=self.device) for _ in range(2)]
            self.u = self.u2[0]
            self.ctl = torch.cuda.Stream(self.device)
            self.gu_sum = torch.zeros((H, head_size), dtype=torch.float32, device=self.device)
            self._calls = 0
            self._tickets = collections.deque()
            self._gu_parts = {}   # (call parity, slices) -> [slices, H, N]: one row per slice, summed in slice order at the end
            p = make_problem(self.slots[0]["r"], self.u, head_size, ydt, variant)
            ck, ws = lib.wkv6_ckpt_bytes(ctypes.byref(p)), lib.wkv6_backward_workspace_bytes(ctypes.byref(p), 1)
            for s in self.slots:
                s["ckpt"] = torch.empty((max(ck, 16),), dtype=torch.uint8, device=self.device)
                s["ws"] = torch.empty((max(ws, 16),), dtype=torch.uint8, device=self.device)
                s["ws_bytes"] = ws

    def slices(self, B: int):
        """The work list: (first row, end row, first head, end head) per slice."""
        H = self.H
        full = [(b0, min(B, b0 + self.rows), 0, H) for b0 in range(0, B, self.rows)]
        if not self.ramp or B == 0:
            return full
        halves = lambda b: [(b, b + 1, 0, H // 2), (b, b + 1, H // 2, H)]
        if B == 1:
            return halves(0)
        return halves(0) + full[1:-1] + halves(B - 1)

    def _copy(self, dev_t, host_t, b0, b1, h0, h1, to_host, stream):
        """One (rows, head group) region between a [B,T,C] host tensor and the slot's compact [rows,T,(h1-h0)*N] buffer."""
        N, T = self.N, self.T
        esz = host_t.element_size()
        assert host_t.stride(2) == 1 and host_t.stride(1) == host_t.shape[2] and host_t.stride(0) == T * host_t.shape[2], \
            "host tensors must be dense [B,T,C]"
        pitch_h, width = host_t.shape[2] * esz, (h1 - h0) * N * esz
        hp = host_t.data_ptr() + (b0 * T * host_t.shape[2] + h0 * N) * esz
        rows = (b1 - b0) * T
        if to_host:
            check(lib.wkv6_copy_2d_async(hp, pitch_h, dev_t.data_ptr(), width, width, rows, 1, stream))
        else:
            check(lib.wkv6_copy_2d_async(dev_t.data_ptr(), width, hp, pitch_h, width, rows, 0, stream))

    def fwd_bwd(self, r, k, v, w, u, gy, out: Optional[Dict[str, torch.Tensor]] = None):
        """r, k, v, w, gy: [B,T,C] host tensors (pinned, so that the copies overlap); u: [H,N] fp32.  Fills / returns
        ``out`` (host tensors y, gr, gk, gv, gw) and returns gu [H,N] fp32 on the host.  Synchronises before returning."""
        return self.wait(self.submit(r, k, v, w, u, gy, out=out))

    def wait(self, ticket):
        """Block until the call that returned ``ticket`` has delivered: (out, gu) with every tensor complete in host memory."""
        done, out, gu_host = ticket
        done.synchronize()
        return out, gu_host

    def submit(self, r, k, v, w, u, gy, out: Optional[Dict[str, torch.Tensor]] = None):
        """``fwd_bwd`` without the final synchronisation: everything is queued and a ticket for ``wait`` comes back.  A loop
        that submits call i + 1 before it waits for call i (with its own ``out`` tensors per call in flight) keeps both copy
        engines busy across the boundary between the calls: the copies back of the last rows of one call run beside the
        copies in of the first rows of the next.  The inputs of a call must stay untouched until its ticket has been waited for."""
        B, T, C = r.shape
        assert T == self.T and C == self.H * self.N
        host = dict(zip(_IN, (r, k, v, w, gy)))
        if out is None:
            out = {n: torch.empty(tuple(r.shape), dtype=self.slots[0][n].dtype).pin_memory() for n in _OUT}
        main = torch.cuda.current_stream(self.device)
        while len(self._tickets) >= 2:   # at most two calls in flight: the u and gu staging buffers are reused after that
            self._tickets.popleft().synchronize()
        ub = self.u2[self._calls & 1]
        gu_host = torch.empty((self.H, self.N), dtype=torch.float32, pin_memory=True)   # this call's own landing buffer
        self._calls += 1
        with torch.cuda.device(self.device):
            work = self.slices(B)
            key = ((self._calls - 1) & 1, len(work))
            if key not in self._gu_parts:
                self._gu_parts[key] = torch.empty((len(work), self.H, self.N), dtype=torch.float32, device=self.device)
            parts = self._gu_parts[key]
            ready = torch.cuda.Event()
            with torch.cuda.stream(self.ctl):
                ub.copy_(u, non_blocking=True)
                parts.zero_()
                ready.record(self.ctl)
            for i, (b0, b1, h0, h1) in enumerate(work):
                n, g = b1 - b0, h1 - h0
                s = self.slots[i % len(self.slots)]
                # the slot's buffers, viewed as dense [n, T, g*N] tensors
                d = {name: s[name].view(-1)[: n * T * g * self.N].view(n, T, g * self.N) for name in _IN + _OUT}
                gu = s["gu"].view(-1)[: n * g * self.N].view(n, g, self.N)
                u_g = ub[h0:h1]
                with torch.cuda.stream(s["stream"]):
                    s["stream"].wait_event(ready)
                    st = _stream(self.device)
                    for name in _IN:
                        self._copy(d[name], host[name], b0, b1, h0, h1, 0, st)
                    p = make_problem(d["r"], u_g, self.N, d["y"].dtype, self.variant)
                    check(lib.wkv6_forward(ctypes.byref(p), _ptr(d["r"]), _ptr(d["k"]), _ptr(d["v"]), _ptr(d["w"]), _ptr(u_g),
                                           _ptr(d["y"]), None, None, 0, None, _ptr(s["ckpt"]), st))
                    check(lib.wkv6_backward(ctypes.byref(p), _ptr(d["r"]), _ptr(d["k"]), _ptr(d["v"]), _ptr(d["w"]), _ptr(u_g),
                                            _ptr(d["gy"]), _ptr(d["gr"]), _ptr(d["gk"]), _ptr(d["gv"]), _ptr(d["gw"]),
                                            _ptr(gu), _ptr(s["ckpt"]), _ptr(s["ws"]), s["ws_bytes"], st))
                    for name in _OUT:
                        self._copy(d[name], out[name], b0, b1, h0, h1, 1, st)
                    torch.sum(gu, dim=0, out=parts[i, h0:h1])   # this slice's row of gu (its head group; the rest stays zero)
            for s in self.slots:
                main.wait_stream(s["stream"])
            torch.sum(parts, dim=0, out=self.gu_sum)   # one reduction over the slices, the same order in every run
            gu_host.copy_(self.gu_sum, non_blocking=True)
            done_all = torch.cuda.Event()
            done_all.record(main)
            self._tickets.append(done_all)
            return done_all, out, gu_host


def fwd_bwd_host(r, k, v, w, u, gy, head_size: int, out=None, device=None, rows_per_slice: int = 1, slots: int = 6,
                 variant: int = _lib.VARIANT_AUTO):
    """One-shot form of ``HostPipeline`` (allocates the device buffers on every call; keep a ``HostPipeline`` for loops)."""
    B, T, C = r.shape
    pipe = HostPipeline(T, C // head_size, head_size, dtype=r.dtype, device=device, rows_per_slice=rows_per_slice, slots=slots,
                        variant=variant)
    return pipe.fwd_bwd(r, k, v, w, u, gy, out=out)
