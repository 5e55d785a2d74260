"""GPU parity tests of the sequential variant, through the C ABI (ctypes) and the torch operator."""
import glob
import os

import numpy as np
import pytest
import torch

from helpers import TOL_BF16, TOL_F32, np_, oracle_all, rounded, scaled_err
from oracle import c_oracle
from oracle import wkv6_oracle as O

pytestmark = pytest.mark.gpu

GOLD = os.path.join(os.path.dirname(__file__), "golden")


@pytest.fixture(scope="module")
def pkg():
    import star_rwkv6_b200 as m
    return m


def run_op(pkg, d, N, dtype, variant, u_dtype=None):
    from star_rwkv6_b200.rwkv_kernel.torch_rwkv_kernel import RWKVKernelOperator
    op = RWKVKernelOperator(N, d["r"].shape[1], variant=variant)
    t = {n: torch.tensor(d[n]).to(dtype).cuda().requires_grad_(True) for n in ("r", "k", "v", "w")}
    u = torch.tensor(d["u"]).to(u_dtype or dtype).cuda().requires_grad_(True)
    y, st = op(t["r"], t["k"], t["v"], t["w"], u)
    assert st is None
    gy = torch.tensor(d["gy"]).to(y.dtype).cuda()
    y.backward(gy)
    torch.cuda.synchronize()
    return dict(y=np_(y), gr=np_(t["r"].grad), gk=np_(t["k"].grad), gv=np_(t["v"].grad), gw=np_(t["w"].grad),
                gu=np_(u.grad))


def check_all(got, ref, tol):
    for n in ("y", "gr", "gk", "gv", "gw", "gu"):
        e = scaled_err(got[n], ref[n])
        assert np.isfinite(got[n]).all(), n
        assert e <= tol, f"{n}: scaled error {e:.3e} > {tol}"


def test_golden_cfg0_f32(pkg):
    g = np.load(os.path.join(GOLD, "demo_cfg0_f32.npz"))
    got = run_op(pkg, g, int(g["head_size"]), torch.float32, "seq")
    check_all(got, g, TOL_F32)


@pytest.mark.parametrize("name", ["demo_small_f64", "demo_t1_f64", "demo_t3_n16_f64", "demo_masked_f64"])
def test_golden_small(pkg, name):
    g = np.load(os.path.join(GOLD, name + ".npz"))
    got = run_op(pkg, g, int(g["head_size"]), torch.float32, "seq")
    check_all(got, g, TOL_F32)


@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(GOLD, "ops_state_*.npz"))),
                         ids=lambda p: os.path.basename(p))
def test_golden_state_api(pkg, path):
    from star_rwkv6_b200.rwkv_kernel.torch_rwkv_kernel import RWKVKernelOperator
    g = np.load(path)
    N = int(g["head_size"])
    op = RWKVKernelOperator(N, g["r"].shape[1], variant="seq")
    t = [torch.tensor(g[n]).cuda() for n in ("r", "k", "v", "w", "u")]
    smap = torch.tensor(g["state_map"]).cuda() if "state_map" in g.files else None
    y, s = op(*t, return_state=True, init_state=torch.tensor(g["init_state"]).cuda(), state_map=smap)
    assert scaled_err(np_(y), g["y"]) <= TOL_F32
    assert scaled_err(np_(s), g["s_out"]) <= TOL_F32
    assert s.shape == g["s_out"].shape


@pytest.mark.parametrize("N", [8, 16, 32, 64])
@pytest.mark.parametrize("T", [1, 2, 3, 31, 32, 33, 100])
def test_shapes_f32(pkg, N, T):
    d = O.make_inputs(2, T, 3, N, seed=100 + T + N)
    check_all(run_op(pkg, d, N, torch.float32, "seq"), oracle_all(d, N), TOL_F32)


@pytest.mark.parametrize("dtype,tol", [(torch.bfloat16, TOL_BF16), (torch.float16, 2e-3)])
def test_half_inputs(pkg, dtype, tol):
    N = 64
    d = O.make_inputs(2, 256, 4, N, seed=7)
    dr = rounded(d, dtype, names=("r", "k", "v", "w", "u") + (("gy",) if dtype == torch.bfloat16 else ()))
    got = run_op(pkg, d, N, dtype, "seq")
    check_all(got, oracle_all(dr, N), tol)
    assert got["y"].dtype == np.float32


def test_bf16_inputs_fp32_u(pkg):
    N = 64
    d = O.make_inputs(1, 128, 2, N, seed=8)
    dr = rounded(d, torch.bfloat16)
    check_all(run_op(pkg, d, N, torch.bfloat16, "seq", u_dtype=torch.float32), oracle_all(dr, N), TOL_BF16)


def test_extreme_decay(pkg):
    # w = -1e9 is how the time-mix layer masks padded steps (rwkv6_model.py:151): decay exactly 1, no NaN
    N = 16
    d = O.make_inputs(2, 40, 2, N, seed=9)
    d["w"][:, 5:9] = -1e9
    d["w"][:, 20] = 1.0
    d["w"][:, 30] = 4.0
    check_all(run_op(pkg, d, N, torch.float32, "seq"), oracle_all(d, N), TOL_F32)


def test_bit_identical_reruns(pkg):
    d = O.make_inputs(2, 96, 2, 64, seed=10)
    a = run_op(pkg, d, 64, torch.float32, "seq")
    b = run_op(pkg, d, 64, torch.float32, "seq")
    for n in a:
        assert np.array_equal(a[n], b[n]), n


def test_head_sharded_view(pkg):
    # a [B,T,C/2] view of a [B,T,C] tensor is expressed by a row stride; results equal the dense run
    N, H = 32, 4
    d = O.make_inputs(2, 50, H, N, seed=11)
    full = {n: torch.tensor(d[n]).cuda() for n in ("r", "k", "v", "w", "gy")}
    u = torch.tensor(d["u"]).cuda()
    lo = slice(0, 2 * N)
    y, _, _ = pkg.forward_raw(*(full[n][..., lo] for n in "rkvw"), u[:2].contiguous(), N, variant=pkg.VARIANT_SEQ)
    ref, _ = O.wkv6_forward(*(d[n][..., lo] for n in "rkvw"), d["u"][:2], N)
    assert scaled_err(np_(y), ref) <= TOL_F32
    g = pkg.backward_raw(*(full[n][..., lo] for n in "rkvw"), u[:2].contiguous(), full["gy"][..., lo], N,
                         variant=pkg.VARIANT_SEQ)
    gref = O.wkv6_backward(*(d[n][..., lo] for n in "rkvw"), d["u"][:2], d["gy"][..., lo], N)
    for a, b in zip(g, gref):
        assert scaled_err(np_(a), b) <= TOL_F32


def test_state_chaining(pkg):
    from star_rwkv6_b200.rwkv_kernel.torch_rwkv_kernel import RWKVKernelOperator
    N = 64
    d = O.make_inputs(2, 80, 2, N, seed=12)
    op = RWKVKernelOperator(N, 80, variant="seq")
    t = {n: torch.tensor(d[n]).cuda() for n in ("r", "k", "v", "w", "u")}
    y, s = op(t["r"], t["k"], t["v"], t["w"], t["u"], return_state=True)
    cut = 33
    y1, s1 = op(*(t[n][:, :cut].contiguous() for n in "rkvw"), t["u"], return_state=True)
    y2, s2 = op(*(t[n][:, cut:].contiguous() for n in "rkvw"), t["u"], return_state=True, init_state=s1)
    assert scaled_err(np_(torch.cat([y1, y2], 1)), np_(y)) <= 1e-5
    assert scaled_err(np_(s2), np_(s)) <= 1e-5
    yo, so = O.wkv6_forward(d["r"], d["k"], d["v"], d["w"], d["u"], N)
    assert scaled_err(np_(s), so) <= TOL_F32


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_empty_inputs(pkg, dtype):
    """No tokens or no sequences: empty outputs, a zero gu, and a final state equal to the (mapped) initial state."""
    from star_rwkv6_b200 import ops
    from star_rwkv6_b200.rwkv_kernel.torch_rwkv_kernel import RWKVKernelOperator
    N, H = 64, 2
    u = torch.randn(H, N, device="cuda")
    for B, T in ((2, 0), (0, 5), (0, 0)):
        z = torch.zeros(B, T, H * N, dtype=dtype, device="cuda")
        y, s, _ = ops.forward_raw(z, z, z, z, u, N, want_state=True)
        assert y.shape == (B, T, H * N) and s.shape == (B, H, N, N) and not s.any()
        gr, gk, gv, gw, gu = ops.backward_raw(z, z, z, z, u, z, N)
        torch.cuda.synchronize()
        assert gr.shape == gw.shape == (B, T, H * N) and gu.shape == (B, H, N) and not gu.any()
    s0 = torch.randn(2, H, N, N, device="cuda")
    z = torch.zeros(2, 0, H * N, dtype=dtype, device="cuda")
    y, s = RWKVKernelOperator(N, 16)(z, z, z, z, u, return_state=True, init_state=s0, state_map=[1, 0])
    assert y.shape == (2, 0, H * N) and torch.equal(s, s0[[1, 0]])
    t = z.clone().requires_grad_(True)
    uu = u.clone().requires_grad_(True)
    y, _ = RWKVKernelOperator(N, 16)(t, t, t, t, uu)
    y.sum().backward()
    assert t.grad.shape == t.shape and not uu.grad.any()


def test_errors(pkg):
    from star_rwkv6_b200.rwkv_kernel.torch_rwkv_kernel import RWKVKernelOperator
    op = RWKVKernelOperator(64, 16)
    z = torch.zeros(1, 4, 64)
    with pytest.raises(AssertionError):
        op(z, z, z, z, torch.zeros(1, 64))           # CPU tensors: no CPU path
    zc = z.cuda()
    with pytest.raises(AssertionError):
        op(zc, zc, zc, zc.half(), torch.zeros(1, 64).cuda())   # mixed dtypes
    op24 = RWKVKernelOperator(24, 16)
    z24 = torch.zeros(1, 4, 48).cuda()
    with pytest.raises(pkg.WKV6Error):
        op24(z24, z24, z24, z24, torch.zeros(2, 24).cuda())    # head size without a kernel
    with pytest.raises(AssertionError):
        op(zc, zc, zc, zc, torch.zeros(1, 64).cuda(), return_state=True,
           init_state=torch.zeros(1, 1, 64, 64).cuda(), state_map=[3])


@pytest.mark.parametrize("dtype,tol", [(torch.float32, TOL_F32), (torch.bfloat16, TOL_BF16)])
def test_decode_steps(pkg, dtype, tol):
    """256-style decode loop in miniature: prefill with return_state, then single-token steps through the operator
    (which routes T == 1 to the streaming decode kernel), against one oracle pass over the whole sequence."""
    from star_rwkv6_b200.rwkv_kernel.torch_rwkv_kernel import RWKVKernelOperator
    from star_rwkv6_b200 import ops
    N, B, H, Tp, Td = 64, 3, 2, 40, 6
    d = O.make_inputs(B, Tp + Td, H, N, seed=33)
    dr = rounded(d, dtype, names=("r", "k", "v", "w")) if dtype != torch.float32 else d
    t = {n: torch.tensor(d[n]).to(dtype).cuda() for n in ("r", "k", "v", "w")}
    u = torch.tensor(d["u"]).cuda()
    op = RWKVKernelOperator(N, Tp + Td)
    y0, state = op(*(t[n][:, :Tp].contiguous() for n in "rkvw"), u, return_state=True)
    state = state.float().contiguous()
    ys = [y0]
    for s in range(Td):
        step = [t[n][:, Tp + s:Tp + s + 1].contiguous() for n in "rkvw"]
        if s % 2 == 0:
            y1, state = op(*step, u, return_state=True, init_state=state)
        else:  # in-place form used by a serving loop
            y1, state = ops.wkv6_decode(*step, u, N, state=state, out_state=state)
        ys.append(y1)
    yo, so = c_oracle.fwd(dr["r"], dr["k"], dr["v"], dr["w"], d["u"], N)
    assert scaled_err(np_(torch.cat(ys, 1)), yo) <= tol
    assert scaled_err(np_(state), so) <= tol
