"""How far inside the tolerances the kernels sit: per tensor (y, gr, gk, gv, gw, gu, final state) the largest error
against the C oracle, scaled by the largest reference value, and the raw largest absolute error.

Cases: the fp32 smoke configuration (sequential kernels), the headline configuration B8 T4096 H32 in bf16 (chunked
kernels; three sampled (batch, head) sequences, each at full length), the 131072-token sequence cut into segments
(two sampled heads), and inputs that force the per-block reference points of the chunked kernels.  The test asserts
the tolerances and writes the table as ``parity_margins.md`` into the run's output folder (the committed copy lives under
``profiles/``), so that a kernel change that spends error budget shows up as a number.
"""
import os

import numpy as np
import pytest
import torch

from helpers import TOL_BF16, TOL_F32, np_, rounded, scaled_err
from oracle import c_oracle, wkv6_oracle as O
from test_gpu_chunk import _strong_decay_inputs
from test_gpu_fullsize import gen, head_slices

pytestmark = pytest.mark.gpu
N = 64
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ROWS = []


def _record(case, name, got, ref, tol):
    got, ref = np.asarray(got, np.float64), np.asarray(ref, np.float64)
    s, raw = scaled_err(got, ref), float(np.abs(got - ref).max())
    ROWS.append((case, name, s, raw, float(np.abs(ref).max()), tol))
    assert s <= tol, f"{case} {name}: {s:.3e} > {tol:g}"


def _sampled(case, d, pairs, y, grads, s_out=None):
    s = head_slices(d, pairs)
    worst = {}
    for i, (b, h) in enumerate(pairs):
        one = {n: s[n][i:i + 1] for n in s}
        u = np_(d["u"][h:h + 1])
        yo, so = c_oracle.fwd(one["r"], one["k"], one["v"], one["w"], u, N)
        ref = c_oracle.bwd(one["r"], one["k"], one["v"], one["w"], u, one["gy"], N)
        sl = slice(h * N, (h + 1) * N)
        pieces = [("y", np_(y[b, :, sl]), yo[0])]
        pieces += [(nm, np_(g[b, :, sl]), w[0]) for nm, g, w in zip(("gr", "gk", "gv", "gw"), grads[:4], ref[:4])]
        pieces.append(("gu", np_(grads[4][b, h]), ref[4][0, 0]))
        if s_out is not None:
            pieces.append(("s_out", np_(s_out[b, h]), so[0, 0]))
        for nm, got, want in pieces:
            worst.setdefault(nm, []).append((got, want))
    for nm, lst in worst.items():   # one row per tensor: the sampled sequences taken together
        _record(case, nm, np.concatenate([g.ravel() for g, _ in lst]), np.concatenate([w.ravel() for _, w in lst]), TOL_BF16)


def test_margins_table():
    import star_rwkv6_b200 as pkg
    from star_rwkv6_b200 import segments as seg
    # fp32, the reference's CPU-runnable configuration (B2 T64 H2)
    d = O.make_inputs(2, 64, 2, N, seed=0)
    t = {n: torch.tensor(d[n]).cuda() for n in ("r", "k", "v", "w", "gy")}
    u = torch.tensor(d["u"]).cuda()
    y, s, _ = pkg.forward_raw(t["r"], t["k"], t["v"], t["w"], u, N, want_state=True)
    g = pkg.backward_raw(t["r"], t["k"], t["v"], t["w"], u, t["gy"], N)
    yo, so = c_oracle.fwd(d["r"], d["k"], d["v"], d["w"], d["u"], N)
    ref = c_oracle.bwd(d["r"], d["k"], d["v"], d["w"], d["u"], d["gy"], N)
    _record("B2 T64 H2 fp32 (sequential)", "y", np_(y), yo, TOL_F32)
    _record("B2 T64 H2 fp32 (sequential)", "s_out", np_(s), so, TOL_F32)
    for nm, a, b in zip(("gr", "gk", "gv", "gw", "gu"), g, ref):
        _record("B2 T64 H2 fp32 (sequential)", nm, np_(a), b, TOL_F32)

    # headline configuration, bf16, chunked kernels
    d = gen(8, 4096, 32, seed=1)
    y, s, ck = pkg.forward_raw(d["r"], d["k"], d["v"], d["w"], d["u"], N, want_state=True, want_ckpt=True)
    g = pkg.backward_raw(d["r"], d["k"], d["v"], d["w"], d["u"], d["gy"], N, ckpt=ck)
    _sampled("B8 T4096 H32 bf16 (chunked), 3 sequences", d, [(0, 0), (3, 17), (7, 31)], y, g, s)
    del d, y, s, ck, g

    # long sequence, eight segments
    d = gen(1, 131072, 32, seed=4)
    be = seg.LibraryBackend(N)
    y, last, ctx = seg.segmented_forward(be, d["r"], d["k"], d["v"], d["w"], d["u"], 8, want_ckpt=True)
    g = seg.segmented_backward(be, ctx, d["r"], d["k"], d["v"], d["w"], d["u"], d["gy"])
    _sampled("B1 T131072 H32 bf16, 8 segments, 2 sequences", d, [(0, 5), (0, 30)], y, (*g[:4], g[4].reshape(1, 32, N)), last)
    del d, y, last, ctx, g

    # per-block reference points (strong decays) and the switch between the two modes
    for kind in ("some_channels", "alternating", "bursts", "borderline", "steady_fast", "front_loaded", "back_loaded", "lopsided"):
        d = _strong_decay_inputs(kind, 2, 448, 2, seed=51)
        t = {n: torch.tensor(d[n]).to(torch.bfloat16).cuda() for n in ("r", "k", "v", "w", "gy")}
        u = torch.tensor(d["u"]).cuda()
        y, s, ck = pkg.forward_raw(t["r"], t["k"], t["v"], t["w"], u, N, want_state=True, want_ckpt=True)
        g = pkg.backward_raw(t["r"], t["k"], t["v"], t["w"], u, t["gy"], N, ckpt=ck)
        dr = rounded(d, torch.bfloat16)
        yo, so = c_oracle.fwd(dr["r"], dr["k"], dr["v"], dr["w"], dr["u"], N)
        ref = c_oracle.bwd(dr["r"], dr["k"], dr["v"], dr["w"], dr["u"], dr["gy"], N)
        case = f"B2 T448 H2 bf16, strong decay '{kind}'"
        _record(case, "y", np_(y), yo, TOL_BF16)
        _record(case, "s_out", np_(s), so, TOL_BF16)
        for nm, a, b in zip(("gr", "gk", "gv", "gw", "gu"), g, ref):
            _record(case, nm, np_(a), b, TOL_BF16)
    torch.cuda.synchronize()

    out_dir = os.path.join(ROOT, "gpurun_out")
    os.makedirs(out_dir, exist_ok=True)
    with open(os.path.join(out_dir, "parity_margins.md"), "w") as f:
        f.write("| case | tensor | max abs err / max abs ref | max abs err | max abs ref | tolerance |\n|---|---|---|---|---|---|\n")
        for case, nm, s_, raw, mx, tol in ROWS:
            f.write(f"| {case} | {nm} | {s_:.2e} | {raw:.2e} | {mx:.2e} | {tol:g} |\n")
