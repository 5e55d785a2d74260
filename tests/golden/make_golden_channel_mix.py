"""Generates tests/golden/channel_mix_act.npz with torch (float64, autograd) from the expressions of the reference source:
``relu_square(x) = ops.square(ops.relu(x))`` (rwkv6_model.py:47-48) and ``o = r * kv`` with ``r = sigmoid(.)``
(rwkv6_model.py:64, :83).  keras / bert4keras3 are not installed here, so the expressions are evaluated with torch.

    python tests/golden/make_golden_channel_mix.py
"""
import os

import numpy as np
import torch

OUT = os.path.dirname(os.path.abspath(__file__))
g = torch.Generator().manual_seed(11)
rnd = lambda *s: torch.randn(*s, generator=g, dtype=torch.float64)
x = (rnd(3, 7, 13) * 2).requires_grad_(True)
gk = rnd(3, 7, 13)
k = torch.square(torch.relu(x))
(k * gk).sum().backward()
r = (rnd(3, 7, 13) * 3).requires_grad_(True)
kv = rnd(3, 7, 13).requires_grad_(True)
go = rnd(3, 7, 13)
o = torch.sigmoid(r) * kv
(o * go).sum().backward()
np.savez_compressed(os.path.join(OUT, "channel_mix_act.npz"), x=x.detach().numpy(), gk=gk.numpy(), k=k.detach().numpy(),
                    gx=x.grad.numpy(), r=r.detach().numpy(), kv=kv.detach().numpy(), go=go.numpy(), o=o.detach().numpy(),
                    gr=r.grad.numpy(), gkv=kv.grad.numpy())
print("channel_mix_act.npz written")
