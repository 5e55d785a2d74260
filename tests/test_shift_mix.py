"""Input stage of the time-mix block (token shift and the interpolations built on it): the oracle against the golden
fixtures on any host; the CUDA kernels and the TimeMixInputs module against the oracle on a GPU (through the C ABI)."""
import glob
import os

import numpy as np
import pytest

from oracle import shift_mix_oracle as S

GOLDEN = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "shift_mix_*.npz")))


@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p) for p in GOLDEN])
def test_oracle_matches_golden(path):
    z = np.load(path)
    close = lambda a, b: np.abs(a - b).max() <= 1e-11 * max(1.0, np.abs(b).max())
    assert len(GOLDEN) >= 2
    assert close(S.mix(z["x"], z["mu"]), z["x_mix"])
    assert close(S.time_mix_inputs(z["x"], z["mu"], z["A"], z["Bk"], z["bias"]), z["out"])
    assert close(S.mix(z["x"], z["m"]), z["out2"])
    gx, gm = S.mix_backward(z["x"], z["m"], z["gout"])
    assert close(gx, z["gx2"]) and close(gm, z["gm2"])


def test_oracle_vector_gradient_by_differences():
    rng = np.random.default_rng(0)
    x, mu, go = rng.standard_normal((2, 6, 8)), rng.random(8), rng.standard_normal((2, 6, 8))
    gx, gmu = S.mix_backward(x, mu, go)
    f = lambda xx, mm: (S.mix(xx, mm) * go).sum()
    e = 1e-6
    for idx in ((0, 0, 0), (1, 5, 7), (0, 3, 2)):
        d = np.zeros_like(x); d[idx] = e
        assert abs((f(x + d, mu) - f(x - d, mu)) / (2 * e) - gx[idx]) < 1e-6
    d = np.zeros(8); d[3] = e
    assert abs((f(x, mu + d) - f(x, mu - d)) / (2 * e) - gmu[3]) < 1e-6


def _scaled_err(got, ref):
    den = np.abs(ref).max()
    return float(np.abs(np.asarray(got, np.float64) - ref).max() / (den if den else 1.0))


@pytest.mark.gpu
@pytest.mark.parametrize("B,T,C,dtype", [(1, 1, 8, "f32"), (2, 5, 16, "f32"), (3, 70, 64, "f32"), (2, 33, 2048, "bf16"),
                                         (1, 257, 512, "bf16"), (2, 64, 128, "f16")])
def test_gpu_kernels_vs_oracle(B, T, C, dtype):
    import torch
    from star_rwkv6_b200 import time_mix_inputs as M
    tdt = {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16}[dtype]
    tol = 1e-5 if dtype == "f32" else 2e-2
    rng = np.random.default_rng(B * 1000 + T)
    x = torch.tensor(rng.standard_normal((B, T, C)), dtype=tdt).cuda()
    mu = torch.tensor(rng.random(C), dtype=torch.float32).cuda()
    m = torch.tensor(rng.standard_normal((5, B, T, C)), dtype=tdt).cuda()
    go1 = torch.tensor(rng.standard_normal((B, T, C)), dtype=tdt).cuda()
    go5 = torch.tensor(rng.standard_normal((5, B, T, C)), dtype=tdt).cuda()
    xn, mn = x.float().cpu().numpy(), m.float().cpu().numpy()
    # vector form
    out = M._shift_mix_fwd(x, mu, True)
    gx, gmu = M._shift_mix_bwd(x, mu, go1, True)
    rgx, rgmu = S.mix_backward(xn, mu.cpu().numpy(), go1.float().cpu().numpy())
    assert _scaled_err(out.float().cpu().numpy(), S.mix(xn, mu.cpu().numpy())) <= tol
    assert _scaled_err(gx.float().cpu().numpy(), rgx) <= tol and _scaled_err(gmu.cpu().numpy(), rgmu) <= tol
    # five tensors
    out5 = M._shift_mix_fwd(x, m, False)
    gx5, gm5 = M._shift_mix_bwd(x, m, go5, False)
    rgx5, rgm5 = S.mix_backward(xn, mn, go5.float().cpu().numpy())
    assert _scaled_err(out5.float().cpu().numpy(), S.mix(xn, mn)) <= tol
    assert _scaled_err(gx5.float().cpu().numpy(), rgx5) <= tol and _scaled_err(gm5.float().cpu().numpy(), rgm5) <= tol
    # bit-identical reruns of the reduced gradient
    assert torch.equal(M._shift_mix_bwd(x, mu, go1, True)[1], gmu)


@pytest.mark.gpu
def test_gpu_module_against_golden():
    import torch
    from star_rwkv6_b200.time_mix_inputs import TimeMixInputs
    z = np.load([p for p in GOLDEN if "ragged" in p][0])
    Bn, T, D = z["x"].shape
    R = z["Bk"].shape[1]
    mod = TimeMixInputs(D, R).cuda()
    with torch.no_grad():
        mod.time_mix_x.copy_(torch.tensor(z["mu"])); mod.dense_a.copy_(torch.tensor(z["A"]))
        mod.dense_b.copy_(torch.tensor(z["Bk"])); mod.bias_b.copy_(torch.tensor(z["bias"]))
    x = torch.tensor(z["x"], dtype=torch.float32).cuda().requires_grad_(True)
    out = mod(x)
    out.backward(torch.tensor(z["gout"], dtype=torch.float32).cuda())
    assert _scaled_err(out.detach().cpu().numpy(), z["out"]) <= 1e-4
    for got, want in ((x.grad, z["gx"]), (mod.time_mix_x.grad, z["gmu"]), (mod.dense_a.grad, z["gA"]),
                      (mod.dense_b.grad, z["gBk"]), (mod.bias_b.grad, z["gbias"])):
        assert _scaled_err(got.cpu().numpy(), want) <= 1e-4
