"""Channel-mix activations (relu_sq, sigmoid_mul): the oracle against the fixture made from the reference's expressions
(CPU), and the kernels + autograd against the oracle (GPU): fp32 1e-5, bf16 / fp16 within the rounding of the output
dtype (2e-2 / 2e-3 of the largest value)."""
import os

import numpy as np
import pytest
import torch

from oracle import channel_mix_oracle as CO


def test_oracle_matches_reference_expressions(golden_dir):
    d = np.load(os.path.join(golden_dir, "channel_mix_act.npz"))
    assert np.abs(CO.relu_sq(d["x"]) - d["k"]).max() <= 1e-13
    assert np.abs(CO.relu_sq_grad(d["x"], d["gk"]) - d["gx"]).max() <= 1e-13
    assert np.abs(CO.sigmoid_mul(d["r"], d["kv"]) - d["o"]).max() <= 1e-13
    gr, gkv = CO.sigmoid_mul_grad(d["r"], d["kv"], d["go"])
    assert np.abs(gr - d["gr"]).max() <= 1e-13 and np.abs(gkv - d["gkv"]).max() <= 1e-13


def _err(got, ref):
    return float(np.abs(got.detach().float().cpu().numpy() - ref).max() / max(np.abs(ref).max(), 1e-30))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2), (torch.float16, 2e-3)])
@pytest.mark.parametrize("shape", [(3, 7, 13), (2, 100, 256), (5,), (4, 33, 7168)])
def test_kernels_and_autograd_vs_oracle(dtype, tol, shape):
    from star_rwkv6_b200.channel_mix_ops import relu_sq, sigmoid_mul
    g = torch.Generator().manual_seed(sum(shape))
    mk = lambda s: (torch.randn(*shape, generator=g) * s).to(dtype)
    x, gk, r, kv, go = mk(2.0), mk(1.0), mk(3.0), mk(1.0), mk(1.0)
    f = lambda t: t.float().numpy().astype(np.float64)
    xd = x.cuda().requires_grad_(True)
    k = relu_sq(xd)
    k.backward(gk.cuda())
    assert _err(k, CO.relu_sq(f(x))) <= tol
    assert _err(xd.grad, CO.relu_sq_grad(f(x), f(gk))) <= tol
    rd, kvd = r.cuda().requires_grad_(True), kv.cuda().requires_grad_(True)
    o = sigmoid_mul(rd, kvd)
    o.backward(go.cuda())
    wr, wkv = CO.sigmoid_mul_grad(f(r), f(kv), f(go))
    assert _err(o, CO.sigmoid_mul(f(r), f(kv))) <= tol
    assert _err(rd.grad, wr) <= tol and _err(kvd.grad, wkv) <= tol


@pytest.mark.gpu
def test_channel_mix_module_matches_framework_expressions():
    """The model's ChannelMix on these kernels against the same block written with framework operations."""
    from star_rwkv6_b200.model import ChannelMix
    torch.manual_seed(0)
    m = ChannelMix(128, 448).cuda()
    x = torch.randn(2, 37, 128, device="cuda", requires_grad=True)
    out = m(x)
    gout = torch.randn_like(out)
    out.backward(gout)
    got = [out.detach(), x.grad.clone()] + [p.grad.clone() for p in m.parameters()]
    x.grad = None
    for p in m.parameters():
        p.grad = None
    xs = torch.nn.functional.pad(x, (0, 0, 1, 0))[:, :-1, :] - x
    k = torch.relu(m.dense_key(x + xs * m.time_mix_k)) ** 2
    ref = torch.sigmoid(m.dense_receptance(x + xs * m.time_mix_r)) * m.dense_value(k)
    ref.backward(gout)
    want = [ref.detach(), x.grad] + [p.grad for p in m.parameters()]
    for a, b in zip(got, want):
        assert float((a - b).abs().max() / b.abs().max()) <= 2e-4
