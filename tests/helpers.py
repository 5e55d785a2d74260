"""Shared helpers of the GPU parity tests."""
import numpy as np
import torch

from oracle import c_oracle, wkv6_oracle as O

# north_star tolerances: fp32 inputs -> max relative error 1e-4; bf16 inputs with fp32 state -> max abs error
# 2e-2 on unit-scale outputs.  Both are applied as  max|got - ref| / max|ref|  per tensor.
TOL_F32 = 1e-4
TOL_BF16 = 2e-2


def scaled_err(got, ref):
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    den = np.abs(ref).max()
    if den == 0:
        return float(np.abs(got).max())
    return float(np.abs(got - ref).max() / den)


def to_dev(d, dtype, names=("r", "k", "v", "w")):
    out = {}
    for n in names:
        out[n] = torch.tensor(d[n]).to(dtype).cuda()
    return out


def rounded(d, dtype, names=("r", "k", "v", "w", "gy")):
    """The inputs as the kernel sees them: rounded to ``dtype`` and upcast again."""
    out = dict(d)
    for n in names:
        if n in d:
            out[n] = torch.tensor(d[n]).to(dtype).to(torch.float32).numpy()
    return out


def oracle_all(d, N, init_state=None, state_map=None):
    y, s = c_oracle.fwd(d["r"], d["k"], d["v"], d["w"], d["u"], N, init_state, state_map)
    gr, gk, gv, gw, gu = c_oracle.bwd(d["r"], d["k"], d["v"], d["w"], d["u"], d["gy"], N)
    return dict(y=y, s=s, gr=gr, gk=gk, gv=gv, gw=gw, gu=gu.sum(0))


def np_(t):
    return t.detach().float().cpu().numpy()
