"""GPU parity tests of the chunked tensor-core variant (bf16 inputs, fp32 state), through the C ABI."""
import numpy as np
import pytest
import torch

from helpers import TOL_BF16, np_, oracle_all, rounded, scaled_err
from oracle import c_oracle, wkv6_oracle as O

pytestmark = pytest.mark.gpu
N = 64


@pytest.fixture(scope="module")
def pkg():
    import star_rwkv6_b200 as m
    return m


def dev_inputs(d):
    t = {n: torch.tensor(d[n]).to(torch.bfloat16).cuda() for n in ("r", "k", "v", "w", "gy")}
    t["u"] = torch.tensor(d["u"]).cuda()
    return t


def status(pkg):
    from star_rwkv6_b200 import _lib
    return _lib.lib.wkv6_device_status()


@pytest.mark.parametrize("B,T,H", [(1, 64, 1), (2, 128, 2), (1, 256, 3), (2, 1000, 2), (1, 1, 1), (1, 65, 2), (3, 4096, 2)])
def test_forward_vs_oracle(pkg, B, T, H):
    d = O.make_inputs(B, T, H, N, seed=T + H)
    t = dev_inputs(d)
    y, s, _ = pkg.forward_raw(t["r"], t["k"], t["v"], t["w"], t["u"], N, want_state=True, variant=pkg.VARIANT_CHUNK)
    torch.cuda.synchronize()
    assert status(pkg) == 0
    dr = rounded(d, torch.bfloat16)
    yo, so = c_oracle.fwd(dr["r"], dr["k"], dr["v"], dr["w"], dr["u"], N)
    assert np.isfinite(np_(y)).all()
    assert scaled_err(np_(y), yo) <= TOL_BF16
    assert scaled_err(np_(s), so) <= TOL_BF16


def test_forward_matches_sequential_kernel(pkg):
    # the two variants see identical bf16 inputs; they differ only by operand rounding inside the chunked one
    d = O.make_inputs(2, 512, 4, N, seed=21)
    t = dev_inputs(d)
    yc, sc, _ = pkg.forward_raw(t["r"], t["k"], t["v"], t["w"], t["u"], N, want_state=True, variant=pkg.VARIANT_CHUNK)
    ys, ss, _ = pkg.forward_raw(t["r"], t["k"], t["v"], t["w"], t["u"], N, want_state=True, variant=pkg.VARIANT_SEQ)
    assert scaled_err(np_(yc), np_(ys)) <= TOL_BF16
    assert scaled_err(np_(sc), np_(ss)) <= TOL_BF16 / 2


def test_state_in_and_map(pkg):
    B, T, H = 3, 200, 2
    d = O.make_inputs(B, T, H, N, seed=22, with_state=True, kinds=2)
    t = dev_inputs(d)
    s_in = torch.tensor(d["init_state"]).cuda()
    smap = torch.tensor(d["state_map"]).cuda()
    y, s, _ = pkg.forward_raw(t["r"], t["k"], t["v"], t["w"], t["u"], N, s_in=s_in, s_map=smap, want_state=True,
                              variant=pkg.VARIANT_CHUNK)
    dr = rounded(d, torch.bfloat16)
    yo, so = c_oracle.fwd(dr["r"], dr["k"], dr["v"], dr["w"], dr["u"], N, d["init_state"], d["state_map"])
    assert scaled_err(np_(y), yo) <= TOL_BF16
    assert scaled_err(np_(s), so) <= TOL_BF16


def test_extreme_decay(pkg):
    # w = -1e9 (masked steps: decay exactly 1) and w far above the benchmark range (decay clamped at e^-10)
    B, T, H = 1, 192, 2
    d = O.make_inputs(B, T, H, N, seed=23)
    d["w"][:, 10:20] = -1e9
    d["w"][:, 70:75] = 3.0
    d["w"][:, 100] = 8.0
    t = dev_inputs(d)
    y, s, _ = pkg.forward_raw(t["r"], t["k"], t["v"], t["w"], t["u"], N, want_state=True, variant=pkg.VARIANT_CHUNK)
    dr = rounded(d, torch.bfloat16)
    yo, so = c_oracle.fwd(dr["r"], dr["k"], dr["v"], dr["w"], dr["u"], N)
    assert np.isfinite(np_(y)).all() and np.isfinite(np_(s)).all()
    assert scaled_err(np_(y), yo) <= TOL_BF16
    assert scaled_err(np_(s), so) <= TOL_BF16


def test_bit_identical_reruns(pkg):
    d = O.make_inputs(2, 320, 2, N, seed=24)
    t = dev_inputs(d)
    a = pkg.forward_raw(t["r"], t["k"], t["v"], t["w"], t["u"], N, want_state=True, variant=pkg.VARIANT_CHUNK)
    b = pkg.forward_raw(t["r"], t["k"], t["v"], t["w"], t["u"], N, want_state=True, variant=pkg.VARIANT_CHUNK)
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])


def test_operator_autograd_bf16(pkg):
    from star_rwkv6_b200.rwkv_kernel.torch_rwkv_kernel import RWKVKernelOperator
    d = O.make_inputs(2, 256, 2, N, seed=25)
    op = RWKVKernelOperator(N, 256)  # AUTO -> chunked for bf16 / N=64
    t = {n: torch.tensor(d[n]).to(torch.bfloat16).cuda().requires_grad_(True) for n in ("r", "k", "v", "w")}
    u = torch.tensor(d["u"]).cuda().requires_grad_(True)
    y, _ = op(t["r"], t["k"], t["v"], t["w"], u)
    y.backward(torch.tensor(d["gy"]).to(torch.bfloat16).cuda())
    ref = oracle_all(rounded(d, torch.bfloat16), N)
    got = dict(y=np_(y), gr=np_(t["r"].grad), gk=np_(t["k"].grad), gv=np_(t["v"].grad), gw=np_(t["w"].grad),
               gu=np_(u.grad))
    for n in got:
        assert scaled_err(got[n], ref[n]) <= TOL_BF16, n
    assert status(pkg) == 0


@pytest.mark.parametrize("B,T,H,with_ckpt", [(1, 64, 1, True), (2, 128, 2, True), (1, 320, 2, False), (2, 1000, 1, True),
                                             (1, 1, 1, True), (1, 65, 1, False), (2, 4096, 2, True),
                                             (1, 80, 1, True), (2, 1008, 2, False), (1, 16, 2, True)])
def test_backward_vs_oracle(pkg, B, T, H, with_ckpt):
    d = O.make_inputs(B, T, H, N, seed=31 + T + H)
    t = dev_inputs(d)
    ckpt = None
    if with_ckpt:
        _, _, ckpt = pkg.forward_raw(t["r"], t["k"], t["v"], t["w"], t["u"], N, want_ckpt=True, variant=pkg.VARIANT_CHUNK)
        assert ckpt is not None
    g = pkg.backward_raw(t["r"], t["k"], t["v"], t["w"], t["u"], t["gy"], N, ckpt=ckpt, variant=pkg.VARIANT_CHUNK)
    torch.cuda.synchronize()
    assert status(pkg) == 0
    dr = rounded(d, torch.bfloat16)
    ref = c_oracle.bwd(dr["r"], dr["k"], dr["v"], dr["w"], dr["u"], dr["gy"], N)
    for name, got, want in zip(("gr", "gk", "gv", "gw", "gu"), g, ref):
        got = np_(got)
        assert np.isfinite(got).all(), name
        if np.abs(want).max() == 0:
            assert np.abs(got).max() == 0, name
        else:
            assert scaled_err(got, want) <= TOL_BF16, f"{name}: {scaled_err(got, want):.3e}"


@pytest.mark.parametrize("T", [160, 100])
def test_head_sharded_view(pkg, T):
    """Half of the heads as [B, T, C/2] views of [B, T, C] tensors (a row stride, as the head split over GPUs passes them):
    equal to the oracle on that half, and bit-equal to a run on contiguous copies.  T = 160 takes the fast backward's
    paired-token tensor maps, T = 100 its natural-order maps."""
    B, H = 2, 4
    d = O.make_inputs(B, T, H, N, seed=77 + T)
    t = dev_inputs(d)
    hs = slice(2 * N, 4 * N)
    views = [t[n][..., hs] for n in ("r", "k", "v", "w")]
    assert not views[0].is_contiguous()
    u = t["u"][2:].contiguous()
    y, _, ck = pkg.forward_raw(*views, u, N, want_ckpt=True, variant=pkg.VARIANT_CHUNK)
    g = pkg.backward_raw(*views, u, t["gy"][..., hs], N, ckpt=ck, variant=pkg.VARIANT_CHUNK)
    yc, _, ckc = pkg.forward_raw(*(x.contiguous() for x in views), u, N, want_ckpt=True, variant=pkg.VARIANT_CHUNK)
    gc = pkg.backward_raw(*(x.contiguous() for x in views), u, t["gy"][..., hs].contiguous(), N, ckpt=ckc, variant=pkg.VARIANT_CHUNK)
    torch.cuda.synchronize()
    assert status(pkg) == 0
    assert torch.equal(y, yc)
    for a, b in zip(g, gc):
        assert torch.equal(a, b)
    dr = rounded(d, torch.bfloat16)
    sub = {n: np.ascontiguousarray(dr[n][..., hs]) for n in ("r", "k", "v", "w", "gy")}
    yo, _ = c_oracle.fwd(sub["r"], sub["k"], sub["v"], sub["w"], dr["u"][2:], N)
    assert scaled_err(np_(y), yo) <= TOL_BF16
    ref = c_oracle.bwd(sub["r"], sub["k"], sub["v"], sub["w"], dr["u"][2:], sub["gy"], N)
    for name, got, want in zip(("gr", "gk", "gv", "gw", "gu"), g, ref):
        assert scaled_err(np_(got), want) <= TOL_BF16, f"{name}: {scaled_err(np_(got), want):.3e}"


def test_backward_extreme_decay(pkg):
    B, T, H = 1, 192, 2
    d = O.make_inputs(B, T, H, N, seed=41)
    d["w"][:, 10:20] = -1e9
    d["w"][:, 70:75] = 3.0
    d["w"][:, 100] = 8.0
    t = dev_inputs(d)
    g = pkg.backward_raw(t["r"], t["k"], t["v"], t["w"], t["u"], t["gy"], N, variant=pkg.VARIANT_CHUNK)
    dr = rounded(d, torch.bfloat16)
    ref = c_oracle.bwd(dr["r"], dr["k"], dr["v"], dr["w"], dr["u"], dr["gy"], N)
    for name, got, want in zip(("gr", "gk", "gv", "gw", "gu"), g, ref):
        assert np.isfinite(np_(got)).all(), name
        assert scaled_err(np_(got), want) <= TOL_BF16, f"{name}: {scaled_err(np_(got), want):.3e}"


def _strong_decay_inputs(kind, B, T, H, seed):
    """Inputs whose chunks take the per-block reference points (total log2 decay of a chunk below -192 in some channel),
    the single reference, or a mix of both inside one sequence."""
    d = O.make_inputs(B, T, H, N, seed=seed)
    rng = np.random.default_rng(seed)
    w = d["w"].reshape(B, T, H, N)
    if kind == "some_channels":      # eight channels of every head decay by 1.5 .. 6.5 bits per step, all the time
        w[..., 3:11] = rng.uniform(0.0, 1.5, size=w[..., 3:11].shape)
    elif kind == "alternating":      # every other 64-token chunk decays strongly in all channels
        for c0 in range(0, T, 128):
            w[:, c0:c0 + 64] = rng.uniform(0.2, 1.2, size=w[:, c0:c0 + 64].shape)
    elif kind == "bursts":           # short clamped bursts at odd offsets, straddling block and chunk borders
        for t0 in range(5, T, 97):
            w[:, t0:t0 + 9, :, ::3] = 4.0
    elif kind == "borderline":       # total decay of a chunk close to the switch-over limit (192 bits over 64 tokens)
        w[...] = np.log(192.0 / 64 / 1.4426950408889634) + rng.uniform(-0.05, 0.05, size=w.shape)
    elif kind == "steady_fast":      # single reference point with factors up to 2^85: products at masked positions overflow
        w[..., ::4] = 0.6 + rng.uniform(-0.02, 0.02, size=w[..., ::4].shape)
    elif kind == "front_loaded":     # the first half of every chunk decays by about 90 bits in some channels, the second mildly
        for c0 in range(0, T, 64):
            w[:, c0:c0 + 32, :, 1::5] = 0.66 + rng.uniform(-0.02, 0.02, size=w[:, c0:c0 + 32, :, 1::5].shape)
    elif kind == "lopsided":         # 115 of a chunk's 137 bits fall on its first 24 tokens: single reference, far from the middle
        for c0 in range(0, T, 64):
            w[:, c0:c0 + 24, :, ::7] = 1.2
    elif kind == "back_loaded":
        for c0 in range(0, T, 64):
            w[:, c0 + 32:c0 + 64, :, 2::5] = 0.66 + rng.uniform(-0.02, 0.02, size=w[:, c0 + 32:c0 + 64, :, 2::5].shape)
    d["w"] = w.reshape(B, T, H * N).astype(np.float32)
    return d


@pytest.mark.parametrize("kind", ["some_channels", "alternating", "bursts", "borderline", "steady_fast", "front_loaded", "back_loaded", "lopsided"])
def test_reference_point_modes(pkg, kind):
    B, T, H = 2, 448, 2
    d = _strong_decay_inputs(kind, B, T, H, seed=51)
    t = dev_inputs(d)
    y, s, ckpt = pkg.forward_raw(t["r"], t["k"], t["v"], t["w"], t["u"], N, want_state=True, want_ckpt=True,
                                 variant=pkg.VARIANT_CHUNK)
    g = pkg.backward_raw(t["r"], t["k"], t["v"], t["w"], t["u"], t["gy"], N, ckpt=ckpt, variant=pkg.VARIANT_CHUNK)
    torch.cuda.synchronize()
    assert status(pkg) == 0
    dr = rounded(d, torch.bfloat16)
    yo, so = c_oracle.fwd(dr["r"], dr["k"], dr["v"], dr["w"], dr["u"], N)
    ref = c_oracle.bwd(dr["r"], dr["k"], dr["v"], dr["w"], dr["u"], dr["gy"], N)
    assert np.isfinite(np_(y)).all() and np.isfinite(np_(s)).all()
    assert scaled_err(np_(y), yo) <= TOL_BF16
    assert scaled_err(np_(s), so) <= TOL_BF16
    for name, got, want in zip(("gr", "gk", "gv", "gw", "gu"), g, ref):
        assert np.isfinite(np_(got)).all(), name
        assert scaled_err(np_(got), want) <= TOL_BF16, f"{kind} {name}: {scaled_err(np_(got), want):.3e}"


def test_general_backward_full_grid(pkg):
    """More (batch, head) sequences than SMs, every one with a channel that decays by 250 bits per chunk: the general
    backward runs in its two-CTAs-per-SM build (smaller problems take the one-per-SM build).  Sampled sequences against
    the oracle."""
    from test_gpu_fullsize import check_sampled
    B, T, H = 5, 192, 32
    g = torch.Generator(device="cuda").manual_seed(61)
    mk = lambda sc: (torch.randn(B, T, H * N, generator=g, device="cuda") * sc).to(torch.bfloat16)
    d = dict(r=mk(0.125), k=mk(0.125), v=mk(0.125), gy=mk(1.0),
             w=(torch.rand(B, T, H * N, generator=g, device="cuda") * 7 - 6))
    d["w"].view(B, T, H, N)[..., 7] = 1.0
    d["w"] = d["w"].to(torch.bfloat16)
    d["u"] = torch.randn(H, N, generator=g, device="cuda") * 0.1
    y, _, ck = pkg.forward_raw(d["r"], d["k"], d["v"], d["w"], d["u"], N, want_ckpt=True, variant=pkg.VARIANT_CHUNK)
    grads = pkg.backward_raw(d["r"], d["k"], d["v"], d["w"], d["u"], d["gy"], N, ckpt=ck, variant=pkg.VARIANT_CHUNK)
    torch.cuda.synchronize()
    assert status(pkg) == 0
    check_sampled(d, [(0, 0), (2, 17), (4, 31)], y, grads)


def test_backward_bit_identical_reruns(pkg):
    d = O.make_inputs(2, 256, 2, N, seed=42)
    t = dev_inputs(d)
    a = pkg.backward_raw(t["r"], t["k"], t["v"], t["w"], t["u"], t["gy"], N, variant=pkg.VARIANT_CHUNK)
    b = pkg.backward_raw(t["r"], t["k"], t["v"], t["w"], t["u"], t["gy"], N, variant=pkg.VARIANT_CHUNK)
    for x, y in zip(a, b):
        assert torch.equal(x, y)


@pytest.mark.parametrize("rows,n", [(8, 2048), (19, 100), (1, 64), (0, 64)])
def test_sum_rows(pkg, rows, n):
    """wkv6_sum_rows (the gu rows of the segments added up) against a float64 sum."""
    import ctypes
    from star_rwkv6_b200 import _lib, ops
    x = torch.randn(rows, n, device="cuda")
    out = torch.full((n,), 7.0, device="cuda")
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    _lib.check(_lib.lib.wkv6_sum_rows(ops._ptr(x) if rows else None, rows, n, ops._ptr(out), st))
    torch.cuda.synchronize()
    want = x.double().sum(0)
    assert (out.double() - want).abs().max().item() <= 1e-5 * max(1.0, want.abs().max().item())


@pytest.mark.parametrize("B,T,H,G", [(1, 512, 2, 2), (2, 1024, 2, 4), (1, 2048, 1, 8)])
def test_segmented_matches_unsplit(pkg, B, T, H, G):
    """Sequences cut into G segments along T (summaries -> scan -> seeded kernels) against the one-piece kernels."""
    from star_rwkv6_b200 import segments as seg
    d = O.make_inputs(B, T, H, N, seed=81 + G)
    t = dev_inputs(d)
    be = seg.LibraryBackend(N)
    y, last, ctx = seg.segmented_forward(be, t["r"], t["k"], t["v"], t["w"], t["u"], G, want_ckpt=True)
    g = seg.segmented_backward(be, ctx, t["r"], t["k"], t["v"], t["w"], t["u"], t["gy"])
    torch.cuda.synchronize()
    assert status(pkg) == 0
    dr = rounded(d, torch.bfloat16)
    yo, so = c_oracle.fwd(dr["r"], dr["k"], dr["v"], dr["w"], dr["u"], N)
    ref = c_oracle.bwd(dr["r"], dr["k"], dr["v"], dr["w"], dr["u"], dr["gy"], N)
    assert scaled_err(np_(y), yo) <= TOL_BF16
    assert scaled_err(np_(last), so) <= TOL_BF16
    for name, got, want in zip(("gr", "gk", "gv", "gw"), g[:4], ref[:4]):
        assert scaled_err(np_(got), want) <= TOL_BF16, f"{name}: {scaled_err(np_(got), want):.3e}"
    assert scaled_err(np_(g[4]), ref[4].sum(0)) <= TOL_BF16
    # and against the unsplit kernels: same inputs, only the association of the state products differs
    y1, s1, ck = pkg.forward_raw(t["r"], t["k"], t["v"], t["w"], t["u"], N, want_state=True, want_ckpt=True, variant=pkg.VARIANT_CHUNK)
    assert scaled_err(np_(y), np_(y1)) <= 1e-2
    assert scaled_err(np_(last), np_(s1)) <= 1e-2   # two bf16 roundings of the operands apart (summary kernel / forward kernel)


@pytest.mark.parametrize("B,T,H,G", [(2, 512, 2, 2), (1, 2048, 2, 8)])
def test_segmented_without_final_state(pkg, B, T, H, G):
    """need_last=False leaves out the summaries no scan reads (last segment forward, first in reverse): the results are
    bit-equal to the full run, whatever the unwritten summary rows hold (they are poisoned with NaN here)."""
    from star_rwkv6_b200 import segments as seg
    d = O.make_inputs(B, T, H, N, seed=85 + G)
    t = dev_inputs(d)
    full = seg.LibraryBackend(N)
    y0, last, ctx0 = seg.segmented_forward(full, t["r"], t["k"], t["v"], t["w"], t["u"], G, want_ckpt=True)
    g0 = seg.segmented_backward(full, ctx0, t["r"], t["k"], t["v"], t["w"], t["u"], t["gy"])
    lean = seg.LibraryBackend(N, reuse_buffers=True)
    for tag in ("fwd", "rev"):   # the buffers the lean run will reuse, filled with NaN beforehand
        lean._buf("sum_state_" + tag, (B * G, H, N, N), torch.float32, t["r"].device).fill_(float("nan"))
        lean._buf("sum_dec_" + tag, (B * G, H, N), torch.float32, t["r"].device).fill_(float("nan"))
    y1, none, ctx1 = seg.segmented_forward(lean, t["r"], t["k"], t["v"], t["w"], t["u"], G, want_ckpt=True, need_last=False)
    g1 = seg.segmented_backward(lean, ctx1, t["r"], t["k"], t["v"], t["w"], t["u"], t["gy"])
    torch.cuda.synchronize()
    assert status(pkg) == 0 and none is None and ctx1["lean"]
    assert torch.equal(y0, y1)
    for a, b in zip(g0[:4], g1[:4]):
        assert torch.equal(a, b)
    assert scaled_err(np_(g1[4]), np_(g0[4])) <= 1e-6


def test_segmented_autograd(pkg):
    from star_rwkv6_b200 import segments as seg
    d = O.make_inputs(1, 1024, 2, N, seed=91)
    t = {n: torch.tensor(d[n]).to(torch.bfloat16).cuda().requires_grad_(True) for n in ("r", "k", "v", "w")}
    u = torch.tensor(d["u"]).cuda().requires_grad_(True)
    y = seg.wkv6_segmented(t["r"], t["k"], t["v"], t["w"], u, N, segments=4)
    y.backward(torch.tensor(d["gy"]).to(torch.bfloat16).cuda())
    ref = oracle_all(rounded(d, torch.bfloat16), N)
    got = dict(y=np_(y), gr=np_(t["r"].grad), gk=np_(t["k"].grad), gv=np_(t["v"].grad), gw=np_(t["w"].grad), gu=np_(u.grad))
    for n in got:
        assert scaled_err(got[n], ref[n]) <= TOL_BF16, n


def test_operator_auto_segments(pkg):
    from star_rwkv6_b200.rwkv_kernel.torch_rwkv_kernel import RWKVKernelOperator
    from star_rwkv6_b200.segments import auto_segments
    assert auto_segments(8, 4096, 32) == 1 and auto_segments(1, 4096, 32) == 8 and auto_segments(1, 131072, 32) == 8
    d = O.make_inputs(1, 2048, 2, N, seed=93)
    op = RWKVKernelOperator(N, 2048, segments="auto")
    t = {n: torch.tensor(d[n]).to(torch.bfloat16).cuda().requires_grad_(True) for n in ("r", "k", "v", "w")}
    u = torch.tensor(d["u"]).cuda().requires_grad_(True)
    y, _ = op(t["r"], t["k"], t["v"], t["w"], u)
    y.backward(torch.tensor(d["gy"]).to(torch.bfloat16).cuda())
    ref = oracle_all(rounded(d, torch.bfloat16), N)
    got = dict(y=np_(y), gr=np_(t["r"].grad), gk=np_(t["k"].grad), gv=np_(t["v"].grad), gw=np_(t["w"].grad), gu=np_(u.grad))
    for n in got:
        assert scaled_err(got[n], ref[n]) <= TOL_BF16, n
