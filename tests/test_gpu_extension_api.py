"""The extension-level drop-in (``star_rwkv6_b200.rwkv_kernel.wkv6_cuda``): the nine functions of the reference's torch
extension (rwkv_kernel/torch_kernel/wkv6_op.cpp:22-60), called the way the reference's autograd function calls them
(torch_rwkv_kernel.py:14-75: caller-allocated outputs, gu per batch row then summed), against the oracle."""
import numpy as np
import pytest
import torch

from helpers import TOL_BF16, TOL_F32, np_, scaled_err
from oracle import wkv6_oracle as O

pytestmark = pytest.mark.gpu

CASES = [("fp32", torch.float32, TOL_F32), ("bf16", torch.bfloat16, TOL_BF16), ("fp16", torch.float16, 2e-3)]


def _inputs(B, T, H, N, dtype, seed):
    d = O.make_inputs(B, T, H, N, seed=seed)
    t = {n: torch.tensor(d[n]).to(dtype).cuda().contiguous() for n in ("r", "k", "v", "w")}
    t["u"] = torch.tensor(d["u"]).to(dtype).cuda().contiguous()
    rd = {n: t[n].float().cpu().numpy().astype(np.float64) for n in t}     # the oracle sees the rounded inputs
    return d, t, rd


@pytest.mark.parametrize("name,dtype,tol", CASES)
@pytest.mark.parametrize("B,T,H", [(2, 70, 2), (1, 256, 3)])
def test_forward_backward_functions(name, dtype, tol, B, T, H):
    from star_rwkv6_b200.rwkv_kernel import wkv6_cuda
    N, C = 64, H * 64
    d, t, rd = _inputs(B, T, H, N, dtype, seed=B + T)
    ydt = torch.float32 if dtype == torch.float16 else dtype
    y = torch.empty(B, T, C, dtype=ydt, device="cuda")
    getattr(wkv6_cuda, f"forward_{name}")(B, T, C, H, t["r"], t["k"], t["v"], t["w"], t["u"], y)
    gy = torch.tensor(d["gy"]).to(ydt).cuda()
    gr, gk, gv, gw = (torch.empty(B, T, C, dtype=ydt, device="cuda") for _ in range(4))
    gu = torch.empty(B, C, dtype=ydt, device="cuda")
    getattr(wkv6_cuda, f"backward_{name}")(B, T, C, H, t["r"], t["k"], t["v"], t["w"], t["u"], gy, gr, gk, gv, gw, gu)
    torch.cuda.synchronize()
    gyd = gy.float().cpu().numpy().astype(np.float64)
    y_o, _ = O.wkv6_forward(rd["r"], rd["k"], rd["v"], rd["w"], rd["u"], N)
    g_o = O.wkv6_backward(rd["r"], rd["k"], rd["v"], rd["w"], rd["u"], gyd, N)
    assert scaled_err(np_(y), y_o) <= tol
    for got, want, nm in zip((gr, gk, gv, gw), g_o[:4], ("gr", "gk", "gv", "gw")):
        assert scaled_err(np_(got), want) <= tol, nm
    assert scaled_err(np_(torch.sum(gu.float(), 0).view(H, N)), g_o[4].sum(0)) <= tol     # torch_rwkv_kernel.py:73


@pytest.mark.parametrize("name,dtype,tol", CASES)
def test_forward_with_state_functions(name, dtype, tol):
    from star_rwkv6_b200.rwkv_kernel import wkv6_cuda
    B, T, H, N = 3, 40, 2, 64
    C = H * N
    d, t, rd = _inputs(B, T, H, N, dtype, seed=7)
    ydt = torch.float32 if dtype == torch.float16 else dtype
    g = torch.Generator().manual_seed(3)
    s = (torch.randn(2, H, N, N, generator=g) * 0.3).cuda()
    s_map = torch.tensor([1, 0, 1], dtype=torch.int64).cuda()
    fn = getattr(wkv6_cuda, f"forward_with_state_{name}")
    for S in (True, False):
        y = torch.empty(B, T, C, dtype=ydt, device="cuda")
        ys = torch.empty(B, H, N, N, dtype=torch.float32, device="cuda")
        fn(B, T, C, H, S, s_map, t["r"], t["k"], t["v"], t["w"], t["u"], s, y, ys)
        torch.cuda.synchronize()
        y_o, s_o = O.wkv6_forward(rd["r"], rd["k"], rd["v"], rd["w"], rd["u"], N,
                                  init_state=np_(s).astype(np.float64) if S else None, state_map=s_map.cpu().numpy() if S else None)
        assert scaled_err(np_(y), y_o) <= tol
        assert scaled_err(np_(ys), s_o) <= tol
