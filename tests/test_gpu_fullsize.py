"""The benchmark configurations at their full sizes, through the C ABI: properties that need no full-size oracle run
(exact chaining, exact batch permutation, linearity) plus the oracle on sampled (batch, head) sequences.

config 1: B8 T4096 H32 N64 bf16 (the headline metric); config 4: B1 T131072 H32 N64 bf16 (long sequence, split along T).
Inputs are generated on the GPU with a fixed seed at the value distributions of the benchmark (r,k,v ~ N(0,1)/8,
w ~ U(-6,1), gy ~ N(0,1), u ~ N(0,0.1))."""
import numpy as np
import pytest
import torch

from helpers import TOL_BF16, np_, scaled_err
from oracle import c_oracle

pytestmark = pytest.mark.gpu
N = 64


@pytest.fixture(scope="module")
def pkg():
    import star_rwkv6_b200 as m
    return m


def gen(B, T, H, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    C = H * N
    mk = lambda s: (torch.randn(B, T, C, generator=g, device="cuda") * s).to(torch.bfloat16)
    d = dict(r=mk(0.125), k=mk(0.125), v=mk(0.125), gy=mk(1.0),
             w=(torch.rand(B, T, C, generator=g, device="cuda") * 7 - 6).to(torch.bfloat16))
    d["u"] = torch.randn(H, N, generator=g, device="cuda") * 0.1
    return d


def head_slices(d, pairs):
    """The sampled (b, h) sequences as a [len(pairs), T, 64] problem for the oracle (one head each)."""
    cut = lambda x: np.stack([np_(x[b, :, h * N:(h + 1) * N]) for b, h in pairs])
    return {n: cut(d[n]) for n in ("r", "k", "v", "w", "gy")}


def check_sampled(d, pairs, y, grads, tol=TOL_BF16):
    """Oracle on each sampled sequence separately (u differs per head)."""
    s = head_slices(d, pairs)
    for i, (b, h) in enumerate(pairs):
        one = {n: s[n][i:i + 1] for n in s}
        u = np_(d["u"][h:h + 1])
        yo, _ = c_oracle.fwd(one["r"], one["k"], one["v"], one["w"], u, N)
        ref = c_oracle.bwd(one["r"], one["k"], one["v"], one["w"], u, one["gy"], N)
        sl = slice(h * N, (h + 1) * N)
        assert scaled_err(np_(y[b, :, sl]), yo[0]) <= tol, f"y ({b},{h})"
        for name, got, want in zip(("gr", "gk", "gv", "gw"), grads[:4], ref[:4]):
            assert scaled_err(np_(got[b, :, sl]), want[0]) <= tol, f"{name} ({b},{h}): {scaled_err(np_(got[b, :, sl]), want[0]):.3e}"
        assert scaled_err(np_(grads[4][b, h]), ref[4][0, 0]) <= tol, f"gu ({b},{h})"


def test_config1_sampled_oracle_and_properties(pkg):
    B, T, H = 8, 4096, 32
    d = gen(B, T, H, seed=1)
    y, s_full, ckpt = pkg.forward_raw(d["r"], d["k"], d["v"], d["w"], d["u"], N, want_state=True, want_ckpt=True)
    grads = pkg.backward_raw(d["r"], d["k"], d["v"], d["w"], d["u"], d["gy"], N, ckpt=ckpt)
    torch.cuda.synchronize()
    from star_rwkv6_b200 import _lib
    assert _lib.lib.wkv6_device_status() == 0
    for t in (y, s_full, *grads):
        assert torch.isfinite(t.float()).all()
    check_sampled(d, [(0, 0), (3, 17), (7, 31)], y, grads)

    # chaining: the second half started from the state of the first reproduces the one-piece run bit for bit
    # (same chunk grid, fp32 state handed over exactly)
    half = T // 2
    cut = lambda x, a, b: x[:, a:b].contiguous()
    y1, s1, _ = pkg.forward_raw(*(cut(d[n], 0, half) for n in ("r", "k", "v", "w")), d["u"], N, want_state=True)
    y2, s2, _ = pkg.forward_raw(*(cut(d[n], half, T) for n in ("r", "k", "v", "w")), d["u"], N, s_in=s1, want_state=True)
    assert torch.equal(torch.cat([y1, y2], 1), y) and torch.equal(s2, s_full)

    # permuting the batch rows permutes the results, bit for bit
    perm = torch.tensor([5, 2, 7, 0, 3, 6, 1, 4], device="cuda")
    yp, _, ckp = pkg.forward_raw(*(d[n][perm].contiguous() for n in ("r", "k", "v", "w")), d["u"], N, want_ckpt=True)
    gp = pkg.backward_raw(*(d[n][perm].contiguous() for n in ("r", "k", "v", "w")), d["u"], d["gy"][perm].contiguous(), N, ckpt=ckp)
    assert torch.equal(yp, y[perm])
    for a, b in zip(gp, grads):
        assert torch.equal(a, b[perm])

    # linearity in v (y) and in gy (gr, gk, gw; gv is linear in gy too): f(2 x) = 2 f(x) exactly in floating point
    y2x, _, _ = pkg.forward_raw(d["r"], d["k"], d["v"] * 2, d["w"], d["u"], N)
    assert torch.equal(y2x.float(), y.float() * 2)
    g2x = pkg.backward_raw(d["r"], d["k"], d["v"], d["w"], d["u"], d["gy"] * 2, N, ckpt=ckpt)
    for a, b in zip(g2x, grads):
        assert torch.equal(a.float(), b.float() * 2)


def test_config4_long_sequence_segmented(pkg):
    from star_rwkv6_b200 import segments as seg
    B, T, H = 1, 131072, 32
    d = gen(B, T, H, seed=4)
    G = seg.auto_segments(B, T, H)
    assert G == 8
    be = seg.LibraryBackend(N)
    y, last, ctx = seg.segmented_forward(be, d["r"], d["k"], d["v"], d["w"], d["u"], G, want_ckpt=True)
    g = seg.segmented_backward(be, ctx, d["r"], d["k"], d["v"], d["w"], d["u"], d["gy"])
    torch.cuda.synchronize()
    from star_rwkv6_b200 import _lib
    assert _lib.lib.wkv6_device_status() == 0
    # gu comes back summed over the batch ([H,N]); B = 1 here
    gu = g[4].reshape(1, H, N)
    check_sampled(d, [(0, 5), (0, 30)], y, (*g[:4], gu))
    # the unsplit kernels agree (different association of the carried state only)
    y1, s1, _ = pkg.forward_raw(d["r"], d["k"], d["v"], d["w"], d["u"], N, want_state=True)
    assert scaled_err(np_(y), np_(y1)) <= 1e-2
    assert scaled_err(np_(last), np_(s1)) <= 1e-2
