"""TEST INFRASTRUCTURE ONLY.  float64 numpy restatement of the input stage of the reference's time-mix block:
TimeShift (rwkv6_model.py:37-44: pad one zero token in front, drop the last, subtract the input) and the
interpolations of TimeMix.call (rwkv6_model.py:135-146), with their gradients in closed form.
Pinned by tests/golden/shift_mix_*.npz (tests/golden/make_golden_shift.py: torch float64 + autograd on the same
expressions as the reference source).  Only tests, __graft_entry__.smoke() and bench.py's CPU legs may import this."""
import numpy as np


def shift(x):
    xs = np.zeros_like(x)
    xs[:, 1:] = x[:, :-1]
    return xs - x


def mix(x, m):
    """x [B,T,C]; m broadcastable to [nmix,B,T,C] or a vector [C] -> out with m's leading shape."""
    x = np.asarray(x, np.float64)
    return x + shift(x) * np.asarray(m, np.float64)


def mix_backward(x, m, gout):
    """Gradients of sum(mix(x, m) * gout) with respect to x and m.  m is [C] (gout [B,T,C]) or [nmix,B,T,C]."""
    x, m, go = np.asarray(x, np.float64), np.asarray(m, np.float64), np.asarray(gout, np.float64)
    xs = shift(x)
    gm_full = go * xs
    gs = go * m                                   # gradient reaching x through the shift term
    if m.ndim == 1:
        gm, gsum, gdirect = gm_full.sum((0, 1)), gs, go
    else:
        gm, gsum, gdirect = gm_full, gs.sum(0), go.sum(0)
    gx = gdirect - gsum
    gx[:, :-1] += gsum[:, 1:]
    return gx, gm


def time_mix_inputs(x, mu, A, Bk, bias):
    """The five mixed inputs [5,B,T,D]: A [D,5R], Bk [5,R,D], bias [5,1,D]."""
    x = np.asarray(x, np.float64)
    Bn, T, D = x.shape
    R = Bk.shape[1]
    x_mix = mix(x, mu)
    h = np.tanh(x_mix.reshape(Bn * T, D) @ np.asarray(A, np.float64)).reshape(Bn * T, 5, R).transpose(1, 0, 2)
    l = h @ np.asarray(Bk, np.float64) + np.asarray(bias, np.float64)
    return mix(x, l.reshape(5, Bn, T, D))
