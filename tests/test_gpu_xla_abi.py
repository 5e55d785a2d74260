"""The XLA legacy custom-call handlers, driven through ctypes with torch device buffers in the reference's
buffer orders (rwkv_kernel/jax_kernel/rwkv_kernels.cu:451-508) and its 28-byte descriptor."""
import ctypes
import struct

import numpy as np
import pytest
import torch

from helpers import TOL_BF16, TOL_F32, np_, rounded, scaled_err
from oracle import c_oracle, wkv6_oracle as O


def test_descriptor_layout():
    from star_rwkv6_b200 import _lib as L
    blob = L.xla_descriptor(3, 40, 128, 2, True, L.BF16, L.F32)
    assert len(blob) == 28
    B, T, C, H, S = struct.unpack_from("<iiii?", blob, 0)
    x_type, y_type = struct.unpack_from("<ii", blob, 20)
    assert (B, T, C, H, S, x_type, y_type) == (3, 40, 128, 2, True, 0, 2)


def _buffers(tensors):
    arr = (ctypes.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])
    return arr


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,code,tol", [(torch.float32, 2, TOL_F32), (torch.bfloat16, 0, TOL_BF16)])
def test_forward_backward_buffers(dtype, code, tol):
    from star_rwkv6_b200 import _lib as L
    B, T, H, N = 2, 96, 2, 64
    d = O.make_inputs(B, T, H, N, seed=61)
    t = {n: torch.tensor(d[n]).to(dtype).cuda() for n in ("r", "k", "v", "w", "u", "gy")}
    y = torch.empty_like(t["r"])
    desc = L.xla_descriptor(B, T, H * N, H, False, code, code)
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert L.lib.wkv6_xla_forward(st, _buffers([t["r"], t["k"], t["v"], t["w"], t["u"], y]), desc, len(desc)) == 0
    g = [torch.empty_like(t["r"]) for _ in range(4)]
    gu = torch.empty((B, H * N), dtype=dtype, device="cuda")
    rc = L.lib.wkv6_xla_backward(st, _buffers([t["r"], t["k"], t["v"], t["w"], t["u"], t["gy"], *g, gu]), desc, len(desc))
    assert rc == 0, L.lib.wkv6_last_error()
    torch.cuda.synchronize()
    dr = rounded(d, dtype, names=("r", "k", "v", "w", "u", "gy"))
    yo, _ = c_oracle.fwd(dr["r"], dr["k"], dr["v"], dr["w"], dr["u"], N)
    go = c_oracle.bwd(dr["r"], dr["k"], dr["v"], dr["w"], dr["u"], dr["gy"], N)
    assert scaled_err(np_(y), yo) <= tol
    for a, b in zip(g, go[:4]):
        assert scaled_err(np_(a), b) <= tol
    assert scaled_err(np_(gu).reshape(B, H, N), go[4]) <= tol
    assert L.lib.wkv6_xla_forward(st, _buffers([y]), desc[:10], 10) == -1   # wrong descriptor size


@pytest.mark.gpu
def test_forward_with_state_buffers():
    from star_rwkv6_b200 import _lib as L
    B, T, H, N = 3, 50, 2, 64
    d = O.make_inputs(B, T, H, N, seed=62, with_state=True, kinds=2)
    t = {n: torch.tensor(d[n]).cuda() for n in ("r", "k", "v", "w", "u")}
    s_in = torch.zeros((B, H, N, N), device="cuda")
    s_in[:2] = torch.tensor(d["init_state"]).cuda()
    smap = torch.tensor(d["state_map"]).cuda()
    y, ys = torch.empty_like(t["r"]), torch.empty((B, H, N, N), device="cuda")
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    desc = L.xla_descriptor(B, T, H * N, H, True, 2, 2)
    bufs = _buffers([smap, t["r"], t["k"], t["v"], t["w"], t["u"], s_in, y, ys])
    assert L.lib.wkv6_xla_forward_with_state(st, bufs, desc, len(desc)) == 0
    torch.cuda.synchronize()
    yo, so = c_oracle.fwd(d["r"], d["k"], d["v"], d["w"], d["u"], N, d["init_state"], d["state_map"])
    assert scaled_err(np_(y), yo) <= TOL_F32 and scaled_err(np_(ys), so) <= TOL_F32
    desc0 = L.xla_descriptor(B, T, H * N, H, False, 2, 2)
    bufs0 = _buffers([t["r"], t["k"], t["v"], t["w"], t["u"], y, ys])
    assert L.lib.wkv6_xla_forward_with_state(st, bufs0, desc0, len(desc0)) == 0
    torch.cuda.synchronize()
    yo, so = c_oracle.fwd(d["r"], d["k"], d["v"], d["w"], d["u"], N)
    assert scaled_err(np_(y), yo) <= TOL_F32 and scaled_err(np_(ys), so) <= TOL_F32


@pytest.mark.gpu
@pytest.mark.parametrize("B,T,H", [(3, 4096, 16), (1, 8192, 24)])
def test_legacy_backward_beyond_the_built_in_scratch(B, T, H):
    """Eleven buffers, bf16, more (token, channel) pairs than the built-in scratch holds: the handler cuts the problem
    into whole rows (first case: 2 + 1) or head groups of a row (second case: 16 + 8 heads); (batch, head) sequences are
    independent, so the result equals the one-call backward of the same kernels bit for bit."""
    import star_rwkv6_b200 as pkg
    from star_rwkv6_b200 import _lib as L
    N = 64
    assert B * T * H * N * 4 > L.lib.wkv6_static_scratch_bytes()
    g = torch.Generator(device="cuda").manual_seed(B + T)
    mk = lambda s: (torch.randn(B, T, H * N, generator=g, device="cuda") * s).to(torch.bfloat16)
    t = dict(r=mk(0.125), k=mk(0.125), v=mk(0.125), gy=mk(1.0),
             w=(torch.rand(B, T, H * N, generator=g, device="cuda") * 7 - 6).to(torch.bfloat16))
    u = (torch.randn(H, N, generator=g, device="cuda") * 0.1).to(torch.bfloat16)
    outs = [torch.empty_like(t["r"]) for _ in range(4)]
    gu = torch.empty((B, H * N), dtype=torch.bfloat16, device="cuda")
    desc = L.xla_descriptor(B, T, H * N, H, False, 0, 0)
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = L.lib.wkv6_xla_backward(st, _buffers([t["r"], t["k"], t["v"], t["w"], u, t["gy"], *outs, gu]), desc, len(desc))
    assert rc == 0, L.lib.wkv6_last_error()
    want = pkg.backward_raw(t["r"], t["k"], t["v"], t["w"], u, t["gy"], N, variant=pkg.VARIANT_SEQ)
    torch.cuda.synchronize()
    for a, b in zip(outs, want[:4]):
        assert torch.equal(a, b)
    assert torch.equal(gu.view(B, H, N), want[4].to(torch.bfloat16))


@pytest.mark.gpu
def test_extended_buffer_orders_at_the_headline_size():
    """wkv_forward_ckpt / wkv_backward_ws at B8 T4096 H32 bf16 (the chunked kernels behind the XLA surface): y and the
    five gradients against the oracle on sampled (batch, head) sequences."""
    from star_rwkv6_b200 import _lib as L
    from test_gpu_fullsize import check_sampled, gen
    B, T, H, N = 8, 4096, 32, 64
    d = gen(B, T, H, seed=2)
    u = d["u"].to(torch.bfloat16)                      # the legacy descriptor gives u the dtype of r, k, v, w
    desc = L.xla_descriptor(B, T, H * N, H, False, 0, 0)
    ck_bytes, ws_bytes = (L.lib.wkv6_xla_buffer_bytes(desc, len(desc), i) for i in (0, 1))
    assert ck_bytes == B * H * (T // 64) * 4096 * 2 and 16 <= ws_bytes <= B * H * 64 * 4
    y = torch.empty_like(d["r"])
    ckpt = torch.empty((B, H, T // 64, 4096), dtype=torch.bfloat16, device="cuda")
    ws = torch.empty((B, H, 64), dtype=torch.int32, device="cuda")
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = L.lib.wkv6_xla_forward_ckpt(st, _buffers([d["r"], d["k"], d["v"], d["w"], u, y, ckpt]), desc, len(desc))
    assert rc == 0, L.lib.wkv6_last_error()
    g = [torch.empty_like(d["r"]) for _ in range(4)]
    gu = torch.empty((B, H, N), dtype=torch.bfloat16, device="cuda")
    rc = L.lib.wkv6_xla_backward_ws(st, _buffers([d["r"], d["k"], d["v"], d["w"], u, d["gy"], ckpt, *g, gu, ws]), desc, len(desc))
    assert rc == 0, L.lib.wkv6_last_error()
    torch.cuda.synchronize()
    assert L.lib.wkv6_device_status() == 0
    d2 = dict(d, u=u.float())
    check_sampled(d2, [(1, 3), (6, 30)], y, (*g, gu.float()))
