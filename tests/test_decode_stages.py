"""Fused element-wise stages of the single-token step.

CPU: a numpy decode loop assembled from the stage oracles reproduces, token by token, the logits of the reference's own
torch model (fixture tests/golden/model_pth_small.npz): this pins the stage oracles.
GPU: every stage kernel against its oracle (fp32: 1e-5 of the largest value; bf16 / fp16 storage: 2e-2), the decode
kernel with the fused GroupNorm + gate, and the model's fused decode path against the plain framework path."""
import os

import numpy as np
import pytest
import torch

from oracle import decode_stages_oracle as so
from oracle import rwkv6_model_oracle as mo

TOL = {torch.float32: 1e-5, torch.bfloat16: 2e-2, torch.float16: 2e-3}
PERM = [3, 1, 2, 0, 4]   # positions of r, k, v, w, g in the .pth order w, k, v, r, g


def scaled(a, b):
    return np.abs(np.asarray(a, np.float64) - b).max() / max(np.abs(b).max(), 1e-30)


def test_oracle_chain(golden_dir):
    z = np.load(os.path.join(golden_dir, "model_pth_small.npz"))
    cfg = {k[4:]: int(z[k]) for k in z.files if k.startswith("cfg_")}
    sd = {k: v.astype(np.float64) for k, v in mo.synthetic_pth(**cfg).items()}
    tokens, logits = z["tokens"], z["logits"]
    B, T = tokens.shape
    D, N, L = cfg["hidden"], cfg["head_size"], cfg["num_layers"]
    H = D // N
    prev_att = [np.zeros((B, D)) for _ in range(L)]
    prev_ffn = [np.zeros((B, D)) for _ in range(L)]
    state = [np.zeros((B, H, N, N)) for _ in range(L)]
    for t in range(T):
        x = so.layer_norm(sd["emb.weight"][tokens[:, t]], sd["blocks.0.ln0.weight"], sd["blocks.0.ln0.bias"], 1e-5)
        for i in range(L):
            a, f = f"blocks.{i}.att.", f"blocks.{i}.ffn."
            xa, xs, (x_mix,) = so.ln_shift_mix(x, sd[f"blocks.{i}.ln1.weight"], sd[f"blocks.{i}.ln1.bias"], 1e-5, prev_att[i],
                                               [sd[a + "time_maa_x"].reshape(-1)])
            prev_att[i] = xa
            R = cfg["mix_rank"]
            w1 = sd[a + "time_maa_w1"].reshape(D, 5, R)[:, PERM].reshape(D, 5 * R)
            bias = np.stack([sd[a + "time_maa_" + c].reshape(-1) for c in "rkvwg"])
            xr, xk, xv, xw, xg = so.lora_mix(x_mix @ w1, sd[a + "time_maa_w2"][PERM], bias, xa, xs)
            r, k, v = xr @ sd[a + "receptance.weight"].T, xk @ sd[a + "key.weight"].T, xv @ sd[a + "value.weight"].T
            w = sd[a + "time_decay"].reshape(-1) + np.tanh(xw @ sd[a + "time_decay_w1"]) @ sd[a + "time_decay_w2"]
            out, state[i] = so.decode_gated(r, k, v, w, sd[a + "time_faaaa"], xg @ sd[a + "gate.weight"].T,
                                            sd[a + "ln_x.weight"].reshape(H, N), sd[a + "ln_x.bias"].reshape(H, N), 64e-5,
                                            state[i], N)
            x = x + out @ sd[a + "output.weight"].T
            _, _, (xk, xr) = so.ln_shift_mix(x, sd[f"blocks.{i}.ln2.weight"], sd[f"blocks.{i}.ln2.bias"], 1e-5, prev_ffn[i],
                                             [sd[f + "time_maa_k"].reshape(-1), sd[f + "time_maa_r"].reshape(-1)])
            prev_ffn[i] = so.layer_norm(x, sd[f"blocks.{i}.ln2.weight"], sd[f"blocks.{i}.ln2.bias"], 1e-5)
            kv = so.relu_sq(xk @ sd[f + "key.weight"].T) @ sd[f + "value.weight"].T
            x = so.sigmoid_mul_add(x, xr @ sd[f + "receptance.weight"].T, kv)
        got = so.layer_norm(x, sd["ln_out.weight"], sd["ln_out.bias"], 1e-5) @ sd["head.weight"].T
        assert np.abs(got - logits[:, t]).max() <= 1e-11 * np.abs(logits).max(), t


def _rnd(g, *shape, dtype=torch.float32, s=1.0):
    return (torch.randn(*shape, generator=g) * s).to(dtype).cuda()


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,D", [(3, 192), (16, 4096), (1, 8192)])
def test_ln_shift_mix(dtype, B, D):
    from star_rwkv6_b200 import decode_stages as ds
    g = torch.Generator().manual_seed(B + D)
    x, prev = _rnd(g, B, D, dtype=dtype), _rnd(g, B, D, dtype=dtype)
    lw, lb = (1 + 0.2 * torch.randn(D, generator=g)).to(dtype).cuda(), _rnd(g, D, dtype=dtype, s=0.1)
    mu0, mu1 = torch.rand(D, generator=g).cuda(), torch.rand(D, generator=g).cuda()
    f = lambda t: t.float().cpu().numpy()
    xa_o, xs_o, (m0_o, m1_o) = so.ln_shift_mix(f(x), f(lw), f(lb), 1e-5, f(prev), [f(mu0), f(mu1)])
    p1 = prev.clone()
    m0, m1, xa, xs = ds.ln_shift_mix(x, lw, lb, 1e-5, p1, mu0, mu1, want_xa_xs=True)
    tol = TOL[dtype]
    for got, want in ((m0, m0_o), (m1, m1_o), (xa, xa_o), (xs, xs_o), (p1, xa_o)):
        assert scaled(f(got), want) <= tol
    p2 = prev.clone()
    m0b, none1, none2, none3 = ds.ln_shift_mix(x, lw, lb, 1e-5, p2, mu0)
    assert none1 is None and none2 is None and none3 is None and torch.equal(m0b, m0) and torch.equal(p2, p1)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("B,D,R", [(3, 192, 8), (16, 4096, 32), (6, 200, 5)])
def test_lora_mix(dtype, B, D, R):
    from star_rwkv6_b200 import decode_stages as ds
    g = torch.Generator().manual_seed(B * D + R)
    h, wb = _rnd(g, B, 5 * R, dtype=dtype), _rnd(g, 5, R, D, dtype=dtype, s=R ** -0.5)
    bias, xa, xs = _rnd(g, 5, 1, D, dtype=dtype, s=0.3), _rnd(g, B, D, dtype=dtype), _rnd(g, B, D, dtype=dtype)
    f = lambda t: t.float().cpu().numpy()
    want = so.lora_mix(f(h), f(wb), f(bias), f(xa), f(xs))[[0, 1, 2, 4, 3]]      # kernel order r, k, v, g, w
    got = ds.lora_mix(h, wb, bias, xa, xs)
    assert scaled(f(got), want) <= TOL[dtype]


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_activations(dtype):
    from star_rwkv6_b200 import decode_stages as ds
    g = torch.Generator().manual_seed(3)
    x, r, kv = _rnd(g, 5, 777, dtype=dtype), _rnd(g, 5, 777, dtype=dtype, s=3.0), _rnd(g, 5, 777, dtype=dtype)
    f = lambda t: t.float().cpu().numpy()
    assert scaled(f(ds.relu_sq(x)), so.relu_sq(f(x))) <= TOL[dtype]
    assert scaled(f(ds.sigmoid_mul_add(x, r, kv)), so.sigmoid_mul_add(f(x), f(r), f(kv))) <= TOL[dtype]
    e = torch.empty(0, 4, dtype=dtype, device="cuda")
    assert ds.relu_sq(e).shape == (0, 4)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_decode_gated(dtype):
    from star_rwkv6_b200 import decode_stages as ds
    B, H, N = 3, 2, 64
    g = torch.Generator().manual_seed(9)
    r, k, v = (_rnd(g, B, H * N, dtype=dtype, s=0.5) for _ in range(3))
    w = (torch.rand(B, H * N, generator=g) * 7 - 6).to(dtype).cuda()
    g_raw = _rnd(g, B, H * N, dtype=dtype, s=2.0)
    u = _rnd(g, H, N, s=0.3)
    scale, offset = (1 + 0.2 * torch.randn(H, N, generator=g)).cuda(), _rnd(g, H, N, s=0.1)
    S = _rnd(g, B, H, N, N, s=0.5)
    f = lambda t: t.float().cpu().numpy()
    want, s_want = so.decode_gated(f(r), f(k), f(v), f(w), f(u), f(g_raw), f(scale), f(offset), 64e-5, f(S), N)
    got = ds.wkv6_decode_gated(r, k, v, w, u, g_raw, scale, offset, 64e-5, N, S)
    assert scaled(f(got), want) <= (1e-4 if dtype == torch.float32 else 2e-2)
    assert scaled(f(S), s_want) <= 1e-5


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_model_fused_decode_matches_plain(dtype):
    from star_rwkv6_b200.model import RWKV6
    torch.manual_seed(1)
    model = RWKV6(3, 211, 256, head_size=64, decomposer_size=8, expand_size=512, decay_rank=16).cuda()
    with torch.no_grad():
        for name, p in model.named_parameters():
            if name.endswith(("time_mix_x", "time_mix_k", "time_mix_r")):
                p.uniform_(0, 1)
            if name.endswith("bias_b"):
                p.normal_(0, 0.3)
    if dtype == torch.bfloat16:
        model.to_bf16_()
    model.eval()
    tok = torch.randint(0, 211, (4, 40), device="cuda")
    _, st_a = model.prefill(tok[:, :24])
    _, st_b = model.prefill(tok[:, :24])
    scale = None
    for t in range(24, 40):
        la = model.decode(tok[:, t:t + 1], st_a, fused=True).float()
        lb = model.decode(tok[:, t:t + 1], st_b, fused=False).float()
        scale = lb.abs().max().item()
        assert (la - lb).abs().max().item() <= (1e-4 if dtype == torch.float32 else 4e-2) * scale, t
    for (xa, Sa), (xb, Sb) in ((a[0], b[0]) for a, b in zip(st_a, st_b)):
        assert (Sa - Sb).abs().max().item() <= (1e-4 if dtype == torch.float32 else 2e-2) * Sb.abs().max().item()
