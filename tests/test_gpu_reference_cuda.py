"""The reference's own CUDA kernels (compiled unchanged for sm_100a into oracle/_ref/, where the reference tree was
at hand) against the oracle: they are the GPU-side baseline the benchmark reports beside this library, so their
results are pinned here first.  Skipped when that library has not been built."""
import numpy as np
import pytest
import torch

from helpers import TOL_BF16, TOL_F32, np_, rounded, scaled_err
from oracle import c_oracle, ref_cuda, wkv6_oracle as O

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not ref_cuda.available(), reason="oracle/_ref/libref_wkv6_cuda.so not built")]


@pytest.mark.parametrize("dtype,tol", [(torch.float32, TOL_F32), (torch.bfloat16, TOL_BF16)])
def test_reference_cuda_kernels_match_the_oracle(dtype, tol):
    B, T, H, N = 2, 96, 2, 64
    d = O.make_inputs(B, T, H, N, seed=7)
    t = {n: torch.tensor(d[n]).to(dtype).cuda() for n in ("r", "k", "v", "w", "u", "gy")}
    y = torch.empty_like(t["r"])
    g = [torch.empty_like(t["r"]) for _ in range(4)]
    gu = torch.empty((B, H * N), dtype=dtype, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    ref_cuda.forward(t["r"], t["k"], t["v"], t["w"], t["u"], y, st)
    ref_cuda.backward(t["r"], t["k"], t["v"], t["w"], t["u"], t["gy"], *g, gu, st)
    torch.cuda.synchronize()
    assert ref_cuda.lib().ref_wkv6_last_cuda_error() == 0
    dr = rounded(d, dtype, names=("r", "k", "v", "w", "u", "gy"))
    yo, _ = c_oracle.fwd(dr["r"], dr["k"], dr["v"], dr["w"], dr["u"], N)
    go = c_oracle.bwd(dr["r"], dr["k"], dr["v"], dr["w"], dr["u"], dr["gy"], N)
    # the reference kernels use the fast-math intrinsic __expf for the decays (rwkv_kernels.cu:125): 1e-3 in fp32
    tol = max(tol, 1e-3)
    assert scaled_err(np_(y), yo) <= tol
    for name, a, b in zip(("gr", "gk", "gv", "gw"), g, go[:4]):
        assert scaled_err(np_(a), b) <= tol, name
    assert scaled_err(np_(gu).reshape(B, H, N), go[4]) <= tol
