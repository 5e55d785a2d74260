"""Output stage of the time-mix block (per-head GroupNorm, then the gate): the oracle against the golden fixtures on
any host, the CUDA kernels against the oracle on a GPU (through the C ABI)."""
import glob
import os

import numpy as np
import pytest

from oracle import gn_gate_oracle as G

GOLDEN = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "gn_gate_*.npz")))


def test_fixtures_present():
    assert len(GOLDEN) >= 3


@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p) for p in GOLDEN])
def test_oracle_matches_golden(path):
    z = np.load(path)
    d = {k: z[k] for k in ("y", "g", "scale", "offset", "gout")}
    out = G.forward(d["y"], d["g"], d["scale"], d["offset"])
    gy, gg, gs, go = G.backward(d["y"], d["g"], d["scale"], d["offset"], d["gout"])
    for got, name in ((out, "out"), (gy, "gy"), (gg, "gg"), (gs, "gscale"), (go, "goffset")):
        want = z["ref_" + name]
        assert np.abs(got - want).max() <= 1e-10 * max(1.0, np.abs(want).max()), name


def test_oracle_edge_cases():
    # a constant head normalises to zero (variance 0: only eps under the root), so out = offset * g
    H, N = 2, 64
    d = G.make_inputs(3, H, N, seed=5)
    d["y"][:] = 0.25
    out = G.forward(d["y"], d["g"], d["scale"], d["offset"])
    assert np.allclose(out, np.tile(d["offset"].reshape(1, -1), (3, 1)) * d["g"], atol=1e-12)


def test_oracle_silu_gate_matches_autograd():
    """The stage with the gate's SiLU inside, pinned on torch float64 autograd over the reference's expressions
    (rwkv6_model.py:147 silu(dense_g(.)), :93-99 GroupNorm, :158-160 the product)."""
    import torch
    H, N, rows = 2, 64, 5
    d = G.make_inputs(rows, H, N, seed=3)
    t = {k: torch.tensor(v, dtype=torch.float64).requires_grad_(k != "gout") for k, v in d.items()}
    xh = torch.nn.functional.layer_norm(t["y"].reshape(rows, H, N), (N,), eps=G.EPSILON)
    out = ((xh * t["scale"] + t["offset"]).reshape(rows, H * N)) * torch.nn.functional.silu(t["g"])
    (out * t["gout"]).sum().backward()
    assert np.abs(G.forward_silu(d["y"], d["g"], d["scale"], d["offset"]) - out.detach().numpy()).max() <= 1e-12
    got = G.backward_silu(d["y"], d["g"], d["scale"], d["offset"], d["gout"])
    for a, b in zip(got, (t["y"].grad, t["g"].grad, t["scale"].grad, t["offset"].grad)):
        assert np.abs(a - b.numpy()).max() <= 1e-10 * max(1.0, float(b.abs().max()))


# ---- GPU parity (bf16: max error relative to max|ref| <= 2e-2; fp32: <= 1e-4, the tolerances of the WKV path) ------

def _scaled_err(got, ref):
    den = np.abs(ref).max()
    return float(np.abs(np.asarray(got, np.float64) - ref).max() / (den if den else 1.0))


@pytest.mark.gpu
@pytest.mark.parametrize("rows,H,dtype", [(1, 1, "f32"), (7, 2, "f32"), (33, 3, "bf16"), (1000, 32, "bf16"), (2048, 64, "bf16"),
                                          (100, 5, "f16"), (4096, 32, "f32")])
def test_gpu_vs_oracle(rows, H, dtype):
    import torch
    from star_rwkv6_b200 import group_norm as M
    N = 64
    tdt = {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16}[dtype]
    tol = 1e-4 if dtype == "f32" else 2e-2
    d = G.make_inputs(rows, H, N, seed=rows + H)
    t = {k: torch.tensor(v).to(tdt).cuda() for k, v in d.items() if k in ("y", "g", "gout")}
    scale, offset = torch.tensor(d["scale"]).cuda(), torch.tensor(d["offset"]).cuda()
    rd = {k: t[k].float().cpu().numpy() for k in t}  # the inputs as the kernel sees them
    out = M.groupnorm_gate_forward_raw(t["y"], t["g"], scale, offset)
    gy, gg, gs, go = M.groupnorm_gate_backward_raw(t["y"], t["g"], scale, offset, t["gout"])
    ref_out = G.forward(rd["y"], rd["g"], d["scale"], d["offset"])
    ref = G.backward(rd["y"], rd["g"], d["scale"], d["offset"], rd["gout"])
    assert _scaled_err(out.float().cpu().numpy(), ref_out) <= tol
    for name, got, want in zip(("gy", "gg", "gscale", "goffset"), (gy, gg, gs, go), ref):
        assert np.isfinite(got.float().cpu().numpy()).all(), name
        assert _scaled_err(got.float().cpu().numpy(), want) <= tol, name


@pytest.mark.gpu
@pytest.mark.parametrize("rows,H,dtype", [(7, 2, "f32"), (1000, 32, "bf16"), (100, 5, "f16")])
def test_gpu_silu_gate_vs_oracle(rows, H, dtype):
    import torch
    from star_rwkv6_b200 import group_norm as M
    N = 64
    tdt = {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16}[dtype]
    tol = 1e-4 if dtype == "f32" else 2e-2
    d = G.make_inputs(rows, H, N, seed=rows + H)
    d["g"] = np.random.default_rng(rows).standard_normal((rows, H * N)).astype(np.float32) * 2   # the raw gate projection
    t = {k: torch.tensor(v).to(tdt).cuda() for k, v in d.items() if k in ("y", "g", "gout")}
    scale, offset = torch.tensor(d["scale"]).cuda(), torch.tensor(d["offset"]).cuda()
    rd = {k: t[k].float().cpu().numpy() for k in t}
    out = M.groupnorm_gate_forward_raw(t["y"], t["g"], scale, offset, gate_is_raw=True)
    got = M.groupnorm_gate_backward_raw(t["y"], t["g"], scale, offset, t["gout"], gate_is_raw=True)
    assert _scaled_err(out.float().cpu().numpy(), G.forward_silu(rd["y"], rd["g"], d["scale"], d["offset"])) <= tol
    for name, a, want in zip(("gy", "gg_raw", "gscale", "goffset"), got, G.backward_silu(rd["y"], rd["g"], d["scale"], d["offset"], rd["gout"])):
        assert _scaled_err(a.float().cpu().numpy(), want) <= tol, name


@pytest.mark.gpu
def test_gpu_module_autograd_and_reruns():
    import torch
    from star_rwkv6_b200.group_norm import GroupNormGate
    H, N, rows = 4, 64, 300
    d = G.make_inputs(rows, H, N, seed=9)
    m = GroupNormGate(H * N, N).cuda()
    with torch.no_grad():
        m.scale.copy_(torch.tensor(d["scale"])); m.offset.copy_(torch.tensor(d["offset"]))
    y = torch.tensor(d["y"]).cuda().reshape(3, 100, H * N).requires_grad_(True)
    g = torch.tensor(d["g"]).cuda().reshape(3, 100, H * N).requires_grad_(True)
    out = m(y, g)
    out.backward(torch.tensor(d["gout"]).cuda().reshape(3, 100, H * N))
    ref = G.backward(d["y"], d["g"], d["scale"], d["offset"], d["gout"])
    assert _scaled_err(out.detach().cpu().numpy().reshape(rows, -1), G.forward(d["y"], d["g"], d["scale"], d["offset"])) <= 1e-4
    for got, want in zip((y.grad, g.grad, m.scale.grad, m.offset.grad), ref):
        assert _scaled_err(got.cpu().numpy().reshape(want.shape), want) <= 1e-4
    # parameter gradients are summed in a fixed order: bit-identical reruns
    from star_rwkv6_b200.group_norm import groupnorm_gate_backward_raw as bw
    a = bw(y.detach(), g.detach(), m.scale.detach(), m.offset.detach(), torch.tensor(d["gout"]).cuda().reshape(3, 100, H * N))
    b = bw(y.detach(), g.detach(), m.scale.detach(), m.offset.detach(), torch.tensor(d["gout"]).cuda().reshape(3, 100, H * N))
    assert all(torch.equal(p, q) for p, q in zip(a, b))


@pytest.mark.gpu
def test_gpu_rejects_bad_arguments():
    import torch
    from star_rwkv6_b200 import WKV6Error
    from star_rwkv6_b200 import group_norm as M
    y = torch.zeros(4, 2 * 32, device="cuda")
    with pytest.raises(WKV6Error):
        M.groupnorm_gate_forward_raw(y, y, torch.ones(2, 32, device="cuda"), torch.zeros(2, 32, device="cuda"))  # head size 32
