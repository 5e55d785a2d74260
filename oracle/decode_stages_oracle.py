"""TEST INFRASTRUCTURE ONLY.  float64 numpy restatement of the element-wise stages of a single-token step of the
reference's RWKV-6 block: the LayerNorm in front of each half (rwkv6_model.py:205-213), the token shift against the
carried previous token and the mixes (:37-44, 128-146), the channel-mix activations (:47-48, 66-70) and the per-head
GroupNorm with the SiLU gate behind the recurrence (:147, 158-160).

Pinned through the whole-model fixture: a decode loop built from these stages must reproduce the logits of the
reference's own torch model (tests/golden/model_pth_small.npz; tests/test_decode_stages.py::test_oracle_chain).
Only tests may import this module.
"""
import numpy as np

from . import gn_gate_oracle, wkv6_oracle


def layer_norm(x, w, b, eps):
    x = np.asarray(x, np.float64)
    mu = x.mean(-1, keepdims=True)
    var = ((x - mu) ** 2).mean(-1, keepdims=True)
    return (x - mu) / np.sqrt(var + eps) * np.asarray(w, np.float64) + np.asarray(b, np.float64)


def ln_shift_mix(x, ln_w, ln_b, eps, prev, mus):
    """Returns (xa, xs, [xa + xs * mu for mu in mus]); the caller carries xa as the next step's ``prev``."""
    xa = layer_norm(x, ln_w, ln_b, eps)
    xs = np.asarray(prev, np.float64) - xa
    return xa, xs, [xa + xs * np.asarray(mu, np.float64) for mu in mus]


def lora_mix(h, wb, bias, xa, xs):
    """h [B, 5R] before tanh, wb [5, R, D], bias [5, D]: out[m] = xa + xs * (bias[m] + tanh(h_m) wb[m])."""
    h = np.asarray(h, np.float64)
    wb = np.asarray(wb, np.float64)
    R = wb.shape[1]
    out = []
    for m in range(5):
        l = np.tanh(h[:, m * R:(m + 1) * R]) @ wb[m] + np.asarray(bias, np.float64).reshape(5, -1)[m]
        out.append(xa + xs * l)
    return np.stack(out)


def relu_sq(x):
    return np.maximum(np.asarray(x, np.float64), 0.0) ** 2


def sigmoid_mul_add(x, r, kv):
    return np.asarray(x, np.float64) + np.asarray(kv, np.float64) / (1.0 + np.exp(-np.asarray(r, np.float64)))


def decode_gated(r, k, v, w, u, g_raw, scale, offset, eps, state, head_size=64):
    """One token: y from the recurrence with the carried state [B,H,N,N], then GroupNorm * silu(g_raw).
    Returns (out [B, C], new state)."""
    B, C = np.shape(r)
    e = lambda t: np.asarray(t, np.float64).reshape(B, 1, C)
    y, s_out = wkv6_oracle.wkv6_forward(e(r), e(k), e(v), e(w), np.asarray(u, np.float64), head_size, init_state=state)
    g = np.asarray(g_raw, np.float64)
    out = gn_gate_oracle.forward(y.reshape(B, C), g / (1.0 + np.exp(-g)), np.asarray(scale, np.float64),
                                 np.asarray(offset, np.float64), eps)
    return out, s_out
