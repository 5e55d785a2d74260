"""The backward entry point that takes no scratch from the caller (wkv6_backward_static_scratch).

It exists for hosts that cannot allocate around the call - e.g. a legacy XLA custom-call handler, which gets only
the buffers XLA planned - so its scratch is an array inside the library.  These tests drive it through the C ABI
and compare it with wkv6_backward (sequential variant, caller workspace) on the same inputs, twice in a row with
different data, because the array is shared by all calls and keeps the previous call's contents.  The file name
sorts last on purpose: a run that stops at the first failure has then already run every other test.
"""
import ctypes

import numpy as np
import pytest
import torch

from helpers import TOL_BF16, TOL_F32, np_, scaled_err
from oracle import wkv6_oracle as O

pytestmark = pytest.mark.gpu


def _call_static(L, ops, t, u, N, ydt):
    r = t["r"]
    B, T, C = r.shape
    p = ops.make_problem(r, u, N, ydt, L.VARIANT_AUTO)  # the entry point ignores the variant field
    outs = [ops._out_like(r, ydt) for _ in range(4)]   # same strides as the inputs (a head-sharded view stays a view)
    gu = torch.empty((B, C // N, N), dtype=torch.float32, device=r.device)
    ptr = lambda x: ctypes.c_void_p(x.data_ptr())
    rc = L.lib.wkv6_backward_static_scratch(ctypes.byref(p), ptr(t["r"]), ptr(t["k"]), ptr(t["v"]), ptr(t["w"]), ptr(u),
                                            ptr(t["gy"]), *(ptr(o) for o in outs), ptr(gu),
                                            ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0, L.lib.wkv6_last_error().decode()
    return (*outs, gu)


@pytest.mark.parametrize("dtype,tol", [(torch.bfloat16, TOL_BF16), (torch.float32, TOL_F32)])
def test_matches_workspace_entry_point_twice(dtype, tol):
    import star_rwkv6_b200 as pkg
    from star_rwkv6_b200 import _lib as L, ops
    N = 64
    for call, (B, T, H, seed) in enumerate([(2, 300, 2, 51), (1, 128, 3, 52)]):
        d = O.make_inputs(B, T, H, N, seed=seed)
        t = {n: torch.tensor(d[n]).to(dtype).cuda() for n in ("r", "k", "v", "w", "gy")}
        u = torch.tensor(d["u"]).cuda()
        ydt = ops.out_dtype(dtype)
        want = pkg.backward_raw(t["r"], t["k"], t["v"], t["w"], u, t["gy"], N, variant=pkg.VARIANT_SEQ)
        got = _call_static(L, ops, t, u, N, ydt)
        torch.cuda.synchronize()
        for name, a, b in zip(("gr", "gk", "gv", "gw", "gu"), got, want):
            assert np.isfinite(np_(a)).all(), (call, name)
            assert scaled_err(np_(a), np_(b)) <= tol, (call, name)
            assert torch.equal(a, b), (call, name)  # same kernels, same order of operations


@pytest.mark.parametrize("dtype,tol", [(torch.bfloat16, TOL_BF16), (torch.float32, TOL_F32)])
def test_head_sharded_view_uses_the_array(dtype, tol):
    """A column range of a wider tensor (row stride > H*N): also in fp32 this path keeps its scratch in the array."""
    import star_rwkv6_b200 as pkg
    from star_rwkv6_b200 import _lib as L, ops
    N, B, T, H = 64, 2, 130, 4
    for call, seed in enumerate((61, 62)):
        d = O.make_inputs(B, T, H, N, seed=seed)
        wide = {n: torch.tensor(d[n]).to(dtype).cuda() for n in ("r", "k", "v", "w", "gy")}
        t = {n: x[:, :, N:3 * N] for n, x in wide.items()}           # heads 1..2 of 4, no copy
        u = torch.tensor(d["u"]).cuda()[1:3].contiguous()
        ydt = ops.out_dtype(dtype)
        want = pkg.backward_raw(t["r"], t["k"], t["v"], t["w"], u, t["gy"], N, variant=pkg.VARIANT_SEQ)
        got = _call_static(L, ops, t, u, N, ydt)
        torch.cuda.synchronize()
        for name, a, b in zip(("gr", "gk", "gv", "gw", "gu"), got, want):
            assert scaled_err(np_(a), np_(b)) <= tol, (call, name)
            assert torch.equal(a, b), (call, name)


def test_rejects_sizes_beyond_the_built_in_scratch():
    from star_rwkv6_b200 import _lib as L
    limit = L.lib.wkv6_static_scratch_bytes()
    assert limit == 32 << 20
    p = L.Problem()
    p.B, p.T, p.H, p.N = 2, 4096, 32, 64      # 16.8 M (token, channel) pairs > 8.4 M
    p.x_dtype = p.y_dtype = L.BF16
    p.u_dtype = p.gu_dtype = p.s_dtype = L.F32
    dummy = torch.zeros(64, device="cuda")
    ptr = ctypes.c_void_p(dummy.data_ptr())
    rc = L.lib.wkv6_backward_static_scratch(ctypes.byref(p), *([ptr] * 11), None)
    assert rc == -3
    msg = L.lib.wkv6_last_error().decode()
    assert "built-in scratch" in msg and "wkv6_backward" in msg
