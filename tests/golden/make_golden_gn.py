"""Generates tests/golden/gn_gate_*.npz: the output stage of the reference's time-mix block evaluated with torch.

The reference computes it with Keras layers (rwkv6_model.py:84-114 GroupNorm = LayerNormalization(epsilon=64e-5) over
the head_size channels of each head + [num_heads, head_size] scale and offset; :158-160 ``x = group_norm(x); x * g``).
keras / bert4keras3 are not installed here, so the same arithmetic is evaluated with torch.nn.functional.layer_norm
(float64) and torch autograd; the fixtures pin oracle/gn_gate_oracle.py.

    python tests/golden/make_golden_gn.py
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle.gn_gate_oracle import EPSILON, make_inputs  # noqa: E402

OUT = os.path.dirname(os.path.abspath(__file__))


def reference(d, H, N):
    t = {k: torch.tensor(v, dtype=torch.float64, requires_grad=(k != "gout")) for k, v in d.items()}
    rows = t["y"].shape[0]
    x = t["y"].reshape(rows, H, N)
    ln = torch.nn.functional.layer_norm(x, (N,), eps=EPSILON)           # LayerNormalization over head_size
    x = t["scale"].reshape(1, H, N) * ln + t["offset"].reshape(1, H, N)  # GroupNorm.call
    out = x.reshape(rows, H * N) * t["g"]                                # TimeMix.call: x * g
    (out * t["gout"]).sum().backward()
    return dict(out=out.detach().numpy(), gy=t["y"].grad.numpy(), gg=t["g"].grad.numpy(),
                gscale=t["scale"].grad.numpy(), goffset=t["offset"].grad.numpy())


for name, rows, H, N, seed in (("small", 7, 2, 64, 1), ("heads3", 33, 3, 64, 2), ("cfg_like", 6, 32, 64, 3)):
    d = make_inputs(rows, H, N, seed)
    ref = reference(d, H, N)
    np.savez_compressed(os.path.join(OUT, f"gn_gate_{name}.npz"), H=H, N=N, **d, **{"ref_" + k: v for k, v in ref.items()})
    print(name, {k: v.shape for k, v in ref.items()})
