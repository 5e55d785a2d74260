"""TEST INFRASTRUCTURE ONLY.  float64 numpy restatement of the output stage of the reference's time-mix block:
``GroupNorm.call`` (rwkv6_model.py:93-99: LayerNormalization(epsilon=64e-5) over the head_size channels of every
head of every token, then scale and offset of shape [num_heads, head_size]) followed by ``x * g``
(rwkv6_model.py:158-160), and its gradients in closed form.

Pinned by tests/golden/gn_gate_*.npz, which tests/golden/make_golden_gn.py generated with torch's own layer_norm and
autograd (the reference's Keras layers cannot be imported here: keras and bert4keras3 are absent).
Only tests, __graft_entry__.smoke() and bench.py's CPU legs may import this module.
"""
import numpy as np

EPSILON = 64 * 1e-5


def forward(y, g, scale, offset, eps=EPSILON):
    H, N = scale.shape
    y64 = np.asarray(y, np.float64).reshape(-1, H, N)
    g64 = np.asarray(g, np.float64).reshape(-1, H, N)
    mean = y64.mean(-1, keepdims=True)
    var = ((y64 - mean) ** 2).mean(-1, keepdims=True)
    xh = (y64 - mean) / np.sqrt(var + eps)
    out = (xh * np.asarray(scale, np.float64) + np.asarray(offset, np.float64)) * g64
    return out.reshape(np.shape(y))


def backward(y, g, scale, offset, gout, eps=EPSILON):
    """Gradients of sum(out * gout) with respect to y, g, scale, offset."""
    H, N = scale.shape
    y64 = np.asarray(y, np.float64).reshape(-1, H, N)
    g64 = np.asarray(g, np.float64).reshape(-1, H, N)
    go = np.asarray(gout, np.float64).reshape(-1, H, N)
    sc, of = np.asarray(scale, np.float64), np.asarray(offset, np.float64)
    mean = y64.mean(-1, keepdims=True)
    var = ((y64 - mean) ** 2).mean(-1, keepdims=True)
    rstd = 1.0 / np.sqrt(var + eps)
    xh = (y64 - mean) * rstd
    gg = go * (xh * sc + of)
    gog = go * g64
    gscale = (gog * xh).sum(0)
    goffset = gog.sum(0)
    dx = gog * sc
    gy = rstd * (dx - dx.mean(-1, keepdims=True) - xh * (dx * xh).mean(-1, keepdims=True))
    return gy.reshape(np.shape(y)), gg.reshape(np.shape(y)), gscale, goffset


def _silu(x):
    x = np.asarray(x, np.float64)
    return x / (1.0 + np.exp(-x))


def forward_silu(y, g_raw, scale, offset, eps=EPSILON):
    """The same stage with the gate's SiLU inside (rwkv6_model.py:147 `g = silu(dense_g(xg))`)."""
    return forward(y, _silu(g_raw), scale, offset, eps)


def backward_silu(y, g_raw, scale, offset, gout, eps=EPSILON):
    """Gradients with respect to y, g_raw, scale, offset."""
    x = np.asarray(g_raw, np.float64)
    s = 1.0 / (1.0 + np.exp(-x))
    gy, gg, gscale, goffset = backward(y, x * s, scale, offset, gout, eps)
    return gy, gg * (s * (1.0 + x * (1.0 - s))).reshape(np.shape(gg)), gscale, goffset


def make_inputs(rows, H, N, seed=0):
    """y with the scale of WKV outputs at the benchmark distributions (std about 0.03), a silu-activated gate,
    scale near one, small offset, unit-variance output gradient."""
    rng = np.random.default_rng(seed)
    y = (rng.standard_normal((rows, H * N)) * 0.03).astype(np.float32)
    pre = rng.standard_normal((rows, H * N))
    g = (pre / (1.0 + np.exp(-pre))).astype(np.float32)
    scale = (1.0 + 0.1 * rng.standard_normal((H, N))).astype(np.float32)
    offset = (0.1 * rng.standard_normal((H, N))).astype(np.float32)
    gout = rng.standard_normal((rows, H * N)).astype(np.float32)
    return dict(y=y, g=g, scale=scale, offset=offset, gout=gout)
