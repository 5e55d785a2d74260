"""CPU tier: the oracle (numpy float64 and its C twin) against every golden
vector produced from the reference's own Python (tests/golden/make_golden.py),
plus the closed-form known answer of the reference's all-ones smoke input
(test_jax.py:12-16)."""
import glob
import os

import numpy as np
import pytest

from oracle import c_oracle, wkv6_oracle as O

GOLD = os.path.join(os.path.dirname(__file__), "golden")
DEMO = sorted(glob.glob(os.path.join(GOLD, "demo_*.npz")))
OPS = sorted(glob.glob(os.path.join(GOLD, "ops_state_*.npz")))


def relerr(a, b):
    return float(np.abs(np.asarray(a, np.float64) - np.asarray(b, np.float64)).max() / max(np.abs(b).max(), 1e-30))


def test_fixture_inventory():
    assert len(DEMO) == 5 and len(OPS) == 5


@pytest.mark.parametrize("path", DEMO, ids=[os.path.basename(p) for p in DEMO])
@pytest.mark.parametrize("impl", ["numpy", "c"])
def test_demo_golden(path, impl):
    g = np.load(path)
    N = int(g["head_size"])
    # fp32 fixtures carry the reference's own fp32 rounding; f64 ones pin the formulas
    tol = 2e-5 if "f32" in path else 1e-11
    if impl == "numpy":
        y, _ = O.wkv6_forward(g["r"], g["k"], g["v"], g["w"], g["u"], N)
        grads = O.wkv6_backward(g["r"], g["k"], g["v"], g["w"], g["u"], g["gy"], N)
    else:
        y, _ = c_oracle.fwd(g["r"], g["k"], g["v"], g["w"], g["u"], N)
        grads = c_oracle.bwd(g["r"], g["k"], g["v"], g["w"], g["u"], g["gy"], N)
    assert relerr(y, g["y"]) < tol
    gr, gk, gv, gw, gu = grads
    for name, mine in (("gr", gr), ("gk", gk), ("gv", gv), ("gw", gw)):
        ref = g[name]
        if np.abs(ref).max() == 0:
            assert np.abs(mine).max() == 0, name
        else:
            assert relerr(mine, ref) < tol, name
    assert relerr(gu.sum(0), g["gu"]) < tol
    assert np.isfinite(y).all() and all(np.isfinite(x).all() for x in grads)


@pytest.mark.parametrize("path", OPS, ids=[os.path.basename(p) for p in OPS])
@pytest.mark.parametrize("impl", ["numpy", "c"])
def test_ops_state_golden(path, impl):
    g = np.load(path)
    N = int(g["head_size"])
    smap = g["state_map"] if "state_map" in g.files else None
    f = O.wkv6_forward if impl == "numpy" else c_oracle.fwd
    y, s = f(g["r"], g["k"], g["v"], g["w"], g["u"], N, init_state=g["init_state"], state_map=smap)
    assert relerr(y, g["y"]) < 1e-11
    assert relerr(s, g["s_out"]) < 1e-11


def test_all_ones_closed_form():
    # r=k=v=u=1, w=-4: y_t = N * (1 + sum_{s<t} d^(t-1-s)), d = exp(-exp(-4))
    B, T, H, N = 1, 16, 1, 8
    one = np.ones((B, T, H * N))
    y, _ = O.wkv6_forward(one, one, one, -4 * one, np.ones((H, N)), N)
    d = np.exp(-np.exp(-4.0))
    want = np.array([N * (1 + sum(d ** (t - 1 - s) for s in range(t))) for t in range(T)])
    assert np.allclose(y[0, :, 0], want, rtol=1e-13)
    assert np.allclose(y, y[:, :, :1])


def test_state_chaining_equals_one_pass():
    d = O.make_inputs(2, 24, 2, 8, seed=11)
    y, s = O.wkv6_forward(d["r"], d["k"], d["v"], d["w"], d["u"], 8)
    cut = 9
    a = {n: d[n][:, :cut] for n in "rkvw"}
    b = {n: d[n][:, cut:] for n in "rkvw"}
    y1, s1 = O.wkv6_forward(a["r"], a["k"], a["v"], a["w"], d["u"], 8)
    y2, s2 = O.wkv6_forward(b["r"], b["k"], b["v"], b["w"], d["u"], 8, init_state=s1)
    assert np.allclose(np.concatenate([y1, y2], 1), y, rtol=1e-12, atol=1e-14)
    assert np.allclose(s2, s, rtol=1e-12, atol=1e-14)


def test_state_map_validation():
    d = O.make_inputs(3, 4, 1, 8, seed=12, with_state=True, kinds=2)
    with pytest.raises(ValueError):
        O.wkv6_forward(d["r"], d["k"], d["v"], d["w"], d["u"], 8, init_state=d["init_state"])
    with pytest.raises(AssertionError):
        O.wkv6_forward(d["r"], d["k"], d["v"], d["w"], d["u"], 8, init_state=d["init_state"],
                       state_map=np.array([0, 1, 2]))
    with pytest.raises(AssertionError):
        O.wkv6_forward(d["r"], d["k"], d["v"], d["w"], d["u"], 8, state_map=np.array([0, 0, 0]))


def test_c_oracle_f32_close_to_f64():
    d = O.make_inputs(2, 64, 2, 64, seed=0)
    a = c_oracle.bwd(d["r"], d["k"], d["v"], d["w"], d["u"], d["gy"], 64)
    b = c_oracle.bwd(d["r"], d["k"], d["v"], d["w"], d["u"], d["gy"], 64, dtype=np.float32)
    for x, y in zip(a, b):
        assert relerr(y, x) < 1e-5
