"""The PyTorch RWKV-6 block built on this package's kernels against the same block written with plain torch operations
(the expressions of rwkv6_model.py, with the WKV recurrence as the explicit loop of rwkv_v6_demo.py:10-43), in fp32 on
a small shape: outputs and every parameter gradient."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def plain_wkv(r, k, v, w, u, N):
    B, T, C = r.shape
    H = C // N
    r, k, v, w = (x.reshape(B, T, H, N) for x in (r, k, v, w))
    S = torch.zeros(B, H, N, N, dtype=r.dtype, device=r.device)
    ys = []
    for t in range(T):
        kv = k[:, t, :, :, None] * v[:, t, :, None, :]
        ys.append(torch.einsum("bhi,bhij->bhj", r[:, t], u[None, :, :, None] * kv + S))
        S = torch.exp(-torch.exp(w[:, t]))[..., None] * S + kv
    return torch.stack(ys, 1).reshape(B, T, C)


def plain_block(blk, x):
    shift = lambda z: torch.nn.functional.pad(z, (0, 0, 1, 0))[:, :-1] - z
    tm, cm = blk.time_mix, blk.channel_mix
    xa = blk.layer_norm_att(x)
    mi = tm.mix_inputs
    xs = shift(xa)
    x_mix = xa + xs * mi.time_mix_x
    R = mi.decomposer_size
    outs = []
    for i in range(5):
        l = torch.tanh(x_mix @ mi.dense_a[:, i * R:(i + 1) * R]) @ mi.dense_b[i] + mi.bias_b[i]
        outs.append(xa + xs * l)
    xr, xk, xv, xw, xg = outs
    r, k, v = tm.dense_r(xr), tm.dense_k(xk), tm.dense_v(xv)
    w = tm.w_b(torch.tanh(tm.w_a(xw)))
    g = torch.nn.functional.silu(tm.dense_g(xg))
    y = plain_wkv(r, k, v, w, tm.time_faaaa, tm.head_size)
    B, T, C = y.shape
    gn = tm.group_norm
    yn = torch.nn.functional.layer_norm(y.reshape(B, T, gn.num_heads, gn.head_size), (gn.head_size,), eps=gn.epsilon)
    yn = (gn.scale * yn + gn.offset).reshape(B, T, C)
    x = x + tm.dense_o(yn * g)
    xf = blk.layer_norm_ffn(x)
    xs = shift(xf)
    kk = torch.relu(cm.dense_key(xf + xs * cm.time_mix_k)) ** 2
    return x + torch.sigmoid(cm.dense_receptance(xf + xs * cm.time_mix_r)) * cm.dense_value(kk)


def test_block_matches_plain_torch():
    from star_rwkv6_b200.model import Block
    torch.manual_seed(0)
    D, N, T, B = 128, 64, 70, 2
    blk = Block(D, N, decomposer_size=8, expand_size=256, decay_rank=16).cuda()
    x = torch.randn(B, T, D, device="cuda")
    gout = torch.randn(B, T, D, device="cuda")
    xa = x.clone().requires_grad_(True)
    blk(xa).backward(gout)
    got = {n: p.grad.clone() for n, p in blk.named_parameters()}
    out_a = blk(xa).detach()
    blk.zero_grad()
    xb = x.clone().requires_grad_(True)
    out_b = plain_block(blk, xb)
    out_b.backward(gout)
    err = lambda a, b: float((a - b).abs().max() / b.abs().max().clamp_min(1e-30))
    assert err(out_a, out_b.detach()) <= 1e-4
    assert err(xa.grad, xb.grad) <= 1e-4
    for n, p in blk.named_parameters():
        assert err(got[n], p.grad) <= 2e-4, n


def test_model_bf16_step_runs_and_loss_decreases():
    from star_rwkv6_b200.model import RWKV6
    torch.manual_seed(1)
    m = RWKV6(num_layers=2, vocabulary_size=512, hidden_size=128, decomposer_size=8, expand_size=256, decay_rank=16).cuda().to_bf16_()
    opt = torch.optim.AdamW(m.parameters(), lr=3e-3)
    tok = torch.randint(0, 512, (2, 129), device="cuda")
    losses = []
    for _ in range(8):
        logits = m(tok[:, :-1])
        loss = torch.nn.functional.cross_entropy(logits.float().reshape(-1, 512), tok[:, 1:].reshape(-1))
        opt.zero_grad(set_to_none=True)
        loss.backward()
        opt.step()
        losses.append(loss.item())
    assert np.isfinite(losses).all() and losses[-1] < losses[0]


def test_prefill_then_decode_matches_full_forward():
    """logits(prompt + n tokens) from one forward pass == prefill(prompt) followed by n single-token decode steps."""
    from star_rwkv6_b200.model import RWKV6
    torch.manual_seed(2)
    V = 300
    m = RWKV6(num_layers=2, vocabulary_size=V, hidden_size=128, decomposer_size=8, expand_size=256, decay_rank=16).cuda()
    tok = torch.randint(0, V, (3, 70), device="cuda")
    with torch.no_grad():
        full = m(tok)                                   # [B, 70, V]
        logits, states = m.prefill(tok[:, :64])
        outs = [logits]
        for t in range(64, 69):
            outs.append(m.decode(tok[:, t:t + 1], states))
    got = torch.cat(outs, 1)                            # positions 63..68
    want = full[:, 63:69]
    assert float((got - want).abs().max() / want.abs().max()) <= 1e-4
