"""Generates tests/golden/shift_mix_*.npz with torch (float64, autograd) from the expressions of the reference source:
TimeShift.call (rwkv6_model.py:40-43: ``ops.pad(inputs, [[0,0],[1,0],[0,0]])[:, :-1, :] - inputs``) and TimeMix.call
(rwkv6_model.py:135-146).  keras / bert4keras3 are not installed here, so the expressions are evaluated with torch.

    python tests/golden/make_golden_shift.py
"""
import os

import numpy as np
import torch

OUT = os.path.dirname(os.path.abspath(__file__))


def timeshift(x):
    return torch.nn.functional.pad(x, (0, 0, 1, 0))[:, :-1, :] - x


for name, B, T, D, R, seed in (("small", 2, 5, 16, 4, 1), ("ragged", 2, 19, 32, 4, 2)):
    g = torch.Generator().manual_seed(seed)
    rnd = lambda *s: torch.randn(*s, generator=g, dtype=torch.float64)
    x = rnd(B, T, D).requires_grad_(True)
    mu = torch.rand(D, generator=g, dtype=torch.float64).requires_grad_(True)
    A = (rnd(D, 5 * R) * D ** -0.5).requires_grad_(True)
    Bk = (rnd(5, R, D) * R ** -0.5).requires_grad_(True)
    bias = (rnd(5, 1, D) * 0.1).requires_grad_(True)
    gout = rnd(5, B, T, D)
    xs = timeshift(x)
    x_mix = x + xs * mu.reshape(1, 1, D)
    outs, ls = [], []
    for i in range(5):                       # the five DecomposerDense: tanh(x_mix A_i) B_i + b_i, then x + x_shift * (.)
        l_i = torch.tanh(x_mix @ A[:, i * R:(i + 1) * R]) @ Bk[i] + bias[i]
        ls.append(l_i)
        outs.append(x + xs * l_i)
    out = torch.stack(outs)
    (out * gout).sum().backward()
    # second fixture content: the plain interpolation with given tensors m (for the kernel-level checks)
    m = rnd(5, B, T, D)
    x2 = x.detach().clone().requires_grad_(True)
    m2 = m.clone().requires_grad_(True)
    out2 = x2 + timeshift(x2) * m2
    (out2 * gout).sum().backward()
    np.savez_compressed(os.path.join(OUT, f"shift_mix_{name}.npz"), x=x.detach().numpy(), mu=mu.detach().numpy(), A=A.detach().numpy(),
                        Bk=Bk.detach().numpy(), bias=bias.detach().numpy(), gout=gout.numpy(), x_mix=x_mix.detach().numpy(),
                        out=out.detach().numpy(), gx=x.grad.numpy(), gmu=mu.grad.numpy(), gA=A.grad.numpy(), gBk=Bk.grad.numpy(),
                        gbias=bias.grad.numpy(), m=m.numpy(), out2=out2.detach().numpy(), gx2=x2.grad.numpy(), gm2=m2.grad.numpy())
    print(name, out.shape)
