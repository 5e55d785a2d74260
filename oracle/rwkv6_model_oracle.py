"""TEST INFRASTRUCTURE, not product code: a float64 numpy restatement of the RWKV-6 language-model forward pass as the
reference's plain-torch model computes it from a ``.pth`` state dict (rwkv_v6_demo.py: RWKV_Tmix_x060 :45-150,
RWKV_CMix_x060 :156-183, Block :189-216, RWKV :223-257), keyed by the ``.pth`` tensor names that the reference's
converter reads (keras_torch_transport.py:44-145).

Pinned: ``tests/golden/model_pth_small.npz`` holds logits of the reference's own ``RWKV`` module (imported from the
reference tree by ``tests/golden/make_golden_model.py``) for the weights of ``synthetic_pth`` and fixed tokens;
``tests/test_weights.py`` checks this restatement against them.

Only tests may import this module.
"""
from __future__ import annotations

import re

import numpy as np

from . import wkv6_oracle

GROUPNORM_EPS = 64e-5   # rwkv_v6_demo.py:100: 1e-5 * head_size_divisor**2 with head_size_divisor = 8
LAYERNORM_EPS = 1e-5    # torch.nn.LayerNorm default, rwkv_v6_demo.py:195-199,239


def synthetic_pth(num_layers=2, hidden=128, head_size=64, vocab=97, mix_rank=32, decay_rank=64, seed=0):
    """A state dict with the names, shapes and value ranges of a trained RWKV-6 ``.pth`` (rwkv_v6_demo.py:62-99 for
    the time-mix parameters), filled from a seeded numpy generator so that it can be rebuilt anywhere."""
    g = np.random.default_rng(seed)
    D, H = hidden, hidden // head_size
    F = int((D * 3.5) // 32 * 32)   # rwkv_v6_demo.py:228
    f32 = np.float32

    def n(*shape, s=1.0):
        return (g.standard_normal(shape) * s).astype(f32)

    def u(*shape, lo=0.0, hi=1.0):
        return g.uniform(lo, hi, shape).astype(f32)

    sd = {"emb.weight": n(vocab, D, s=0.5), "head.weight": n(vocab, D, s=D ** -0.5),
          "ln_out.weight": u(D, lo=0.5, hi=1.5), "ln_out.bias": n(D, s=0.1),
          "blocks.0.ln0.weight": u(D, lo=0.5, hi=1.5), "blocks.0.ln0.bias": n(D, s=0.1)}
    for i in range(num_layers):
        p = f"blocks.{i}."
        for ln in ("ln1", "ln2"):
            sd[p + ln + ".weight"] = u(D, lo=0.5, hi=1.5)
            sd[p + ln + ".bias"] = n(D, s=0.1)
        a = p + "att."
        for name in ("x", "w", "k", "v", "r", "g"):
            sd[a + "time_maa_" + name] = u(1, 1, D)
        sd[a + "time_maa_w1"] = n(D, 5 * mix_rank, s=D ** -0.5)
        sd[a + "time_maa_w2"] = n(5, mix_rank, D, s=0.3 * mix_rank ** -0.5)
        sd[a + "time_decay"] = u(1, 1, D, lo=-6.0, hi=-0.5)
        sd[a + "time_decay_w1"] = n(D, decay_rank, s=D ** -0.5)
        sd[a + "time_decay_w2"] = n(decay_rank, D, s=0.5 * decay_rank ** -0.5)
        sd[a + "time_faaaa"] = n(H, head_size, s=0.3)
        for name in ("receptance", "key", "value", "gate", "output"):
            sd[a + name + ".weight"] = n(D, D, s=D ** -0.5)
        sd[a + "ln_x.weight"] = u(D, lo=0.5, hi=1.5)
        sd[a + "ln_x.bias"] = n(D, s=0.1)
        f = p + "ffn."
        sd[f + "time_maa_k"] = u(1, 1, D)
        sd[f + "time_maa_r"] = u(1, 1, D)
        sd[f + "key.weight"] = n(F, D, s=D ** -0.5)
        sd[f + "receptance.weight"] = n(D, D, s=D ** -0.5)
        sd[f + "value.weight"] = n(D, F, s=F ** -0.5)
    return sd


def num_layers_of(sd) -> int:
    """keras_torch_transport.py:32-39: highest ``blocks.<i>.`` index + 1."""
    n = 0
    for key in sd:
        m = re.match(r"^blocks\.(\d+)\.", key)
        if m:
            n = max(n, int(m.group(1)) + 1)
    return n


def _layer_norm(x, w, b, eps=LAYERNORM_EPS):
    mu = x.mean(-1, keepdims=True)
    var = ((x - mu) ** 2).mean(-1, keepdims=True)
    return (x - mu) / np.sqrt(var + eps) * w + b


def _shift(x):
    """nn.ZeroPad2d((0, 0, 1, -1)) (rwkv_v6_demo.py:93): the previous token, zeros in front of the first."""
    out = np.zeros_like(x)
    out[:, 1:] = x[:, :-1]
    return out


def _sigmoid(x):
    return 1.0 / (1.0 + np.exp(-x))


def time_mix(sd, prefix, x, head_size):
    """rwkv_v6_demo.py:102-150."""
    P = lambda name: np.asarray(sd[prefix + name], dtype=np.float64)
    B, T, C = x.shape
    H = C // head_size
    xx = _shift(x) - x
    xxx = x + xx * P("time_maa_x")
    xxx = np.tanh(xxx.reshape(B * T, C) @ P("time_maa_w1")).reshape(B * T, 5, -1).transpose(1, 0, 2)
    xxx = np.matmul(xxx, P("time_maa_w2")).reshape(5, B, T, C)
    mw, mk, mv, mr, mg = xxx
    xw = x + xx * (P("time_maa_w") + mw)
    xk = x + xx * (P("time_maa_k") + mk)
    xv = x + xx * (P("time_maa_v") + mv)
    xr = x + xx * (P("time_maa_r") + mr)
    xg = x + xx * (P("time_maa_g") + mg)
    r = xr @ P("receptance.weight").T
    k = xk @ P("key.weight").T
    v = xv @ P("value.weight").T
    gl = xg @ P("gate.weight").T
    g = gl * _sigmoid(gl)
    w = P("time_decay") + np.tanh(xw @ P("time_decay_w1")) @ P("time_decay_w2")
    y, _ = wkv6_oracle.wkv6_forward(r, k, v, w, P("time_faaaa"), head_size)
    yh = y.reshape(B * T, H, head_size)
    mu = yh.mean(-1, keepdims=True)
    var = ((yh - mu) ** 2).mean(-1, keepdims=True)
    yn = ((yh - mu) / np.sqrt(var + GROUPNORM_EPS)).reshape(B, T, C) * P("ln_x.weight") + P("ln_x.bias")
    return (yn * g) @ P("output.weight").T


def channel_mix(sd, prefix, x):
    """rwkv_v6_demo.py:174-183."""
    P = lambda name: np.asarray(sd[prefix + name], dtype=np.float64)
    xx = _shift(x) - x
    xk = x + xx * P("time_maa_k")
    xr = x + xx * P("time_maa_r")
    k = np.maximum(xk @ P("key.weight").T, 0.0) ** 2
    return _sigmoid(xr @ P("receptance.weight").T) * (k @ P("value.weight").T)


def forward(sd, tokens, head_size=64):
    """Logits [B, T, vocab] of the model (rwkv_v6_demo.py:203-216, 244-257)."""
    P = lambda name: np.asarray(sd[name], dtype=np.float64)
    x = P("emb.weight")[np.asarray(tokens)]
    for i in range(num_layers_of(sd)):
        p = f"blocks.{i}."
        if i == 0:
            x = _layer_norm(x, P(p + "ln0.weight"), P(p + "ln0.bias"))
        x = x + time_mix(sd, p + "att.", _layer_norm(x, P(p + "ln1.weight"), P(p + "ln1.bias")), head_size)
        x = x + channel_mix(sd, p + "ffn.", _layer_norm(x, P(p + "ln2.weight"), P(p + "ln2.bias")))
    x = _layer_norm(x, P("ln_out.weight"), P("ln_out.bias"))
    return x @ P("head.weight").T
