"""Randomised shapes and decay regimes: the chunked tensor-core kernels against the C oracle.

Every case draws B, T, H and, per channel, a base value of w between -6 and 1.6 (so that chunks on both sides of the
switch between the single reference and the per-block reference points occur, often inside one sequence), token noise
on top, and now and then a run of tokens with a different decay.  The tolerance is the bf16 one of the other parity
tests.  The seeds are fixed: a failure names its case.
"""
import numpy as np
import pytest
import torch

from helpers import TOL_BF16, np_, rounded, scaled_err
from oracle import c_oracle, wkv6_oracle as O

pytestmark = pytest.mark.gpu
N = 64


def _case(seed):
    rng = np.random.default_rng(1000 + seed)
    B = int(rng.integers(1, 3))
    H = int(rng.integers(1, 4))
    T = int(rng.choice([int(rng.integers(1, 64)), 64, int(rng.integers(65, 400)), 16 * int(rng.integers(1, 40)),
                        64 * int(rng.integers(1, 9)), int(rng.integers(400, 900))]))
    d = O.make_inputs(B, T, H, N, seed=2000 + seed)
    w = d["w"].reshape(B, T, H, N).copy()
    regime = seed % 4
    if regime >= 1:     # per-channel base decays, up to 6.6 bits per token, with token noise
        hi = [0.5, 0.9, 1.6][regime - 1]
        base = rng.uniform(-6.0, hi, size=(1, 1, H, N))
        w = base + rng.normal(0.0, 0.25, size=w.shape)
    if seed % 3 == 0:   # a run of tokens with another decay, at an odd offset
        t0 = int(rng.integers(0, max(1, T - 1)))
        w[:, t0:t0 + int(rng.integers(1, 90)), :, ::int(rng.integers(1, 5))] = rng.uniform(-8.0, 2.5)
    d["w"] = w.reshape(B, T, H * N).astype(np.float32)
    return B, T, H, d


@pytest.mark.parametrize("seed", list(range(24)))
def test_random_case(seed):
    import star_rwkv6_b200 as pkg
    from star_rwkv6_b200 import _lib
    B, T, H, d = _case(seed)
    t = {n: torch.tensor(d[n]).to(torch.bfloat16).cuda() for n in ("r", "k", "v", "w", "gy")}
    u = torch.tensor(d["u"]).cuda()
    y, s, ck = pkg.forward_raw(t["r"], t["k"], t["v"], t["w"], u, N, want_state=True, want_ckpt=True, variant=pkg.VARIANT_CHUNK)
    g = pkg.backward_raw(t["r"], t["k"], t["v"], t["w"], u, t["gy"], N, ckpt=ck, variant=pkg.VARIANT_CHUNK)
    torch.cuda.synchronize()
    assert _lib.lib.wkv6_device_status() == 0
    dr = rounded(d, torch.bfloat16)
    yo, so = c_oracle.fwd(dr["r"], dr["k"], dr["v"], dr["w"], dr["u"], N)
    ref = c_oracle.bwd(dr["r"], dr["k"], dr["v"], dr["w"], dr["u"], dr["gy"], N)
    tag = f"seed {seed}: B{B} T{T} H{H}"
    assert np.isfinite(np_(y)).all() and np.isfinite(np_(s)).all(), tag
    assert scaled_err(np_(y), yo) <= TOL_BF16, f"{tag} y {scaled_err(np_(y), yo):.3e}"
    assert scaled_err(np_(s), so) <= TOL_BF16, f"{tag} s {scaled_err(np_(s), so):.3e}"
    for name, got, want in zip(("gr", "gk", "gv", "gw", "gu"), g, ref):
        got = np_(got)
        assert np.isfinite(got).all(), f"{tag} {name}"
        if np.abs(want).max() == 0:
            assert np.abs(got).max() == 0, f"{tag} {name}"
        else:
            assert scaled_err(got, want) <= TOL_BF16, f"{tag} {name} {scaled_err(got, want):.3e}"
