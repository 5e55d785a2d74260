"""Generate the golden vectors under tests/golden/ by running the reference's own Python.

Run once, where a checkout of the reference exists (its path in the REFERENCE_ROOT
environment variable):

    REFERENCE_ROOT=<checkout of infiy-quine/STAR-RWKV6> python tests/golden/make_golden.py

Two reference code paths are executed unmodified:

* ``rwkv_v6_demo.RWKV_Kernel`` (rwkv_v6_demo.py:10-43) with torch autograd for
  the gradients, as deprecated_code/wkv_torch.py:56 does.
* ``rwkv_kernel/ops_rwkv_kernal.py`` ``RWKVKernelOperator.__call__`` (:28-97) for
  the init_state / state_map / returned-state API.  Its only import,
  ``bert4keras3.backend`` (not installable here), is satisfied by a small
  torch-backed stand-in defined below that provides exactly the ``ops`` names
  the file uses; the operator file itself is loaded from the reference tree.

The resulting ``.npz`` files hold inputs and outputs; the test-suite never
needs the reference checkout.
"""
import importlib.util
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(os.path.dirname(HERE))
REF = os.environ.get("REFERENCE_ROOT") or os.path.join(os.path.dirname(REPO), "reference")
sys.path.insert(0, REPO)

from oracle.wkv6_oracle import make_inputs  # noqa: E402


def _load(path, name):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _backend_stand_in():
    ops = types.SimpleNamespace(
        int64=torch.int64, int32=torch.int32,
        reshape=lambda x, s: torch.reshape(x, tuple(s)),
        zeros=lambda shape, dtype=None: torch.zeros(tuple(shape), dtype=dtype),
        exp=torch.exp,
        stack=lambda xs, axis=0: torch.stack(xs, dim=axis),
        take=lambda x, idx, axis=0: torch.index_select(x, axis, idx),
        cast=lambda x, dt: x.to(dt),
        convert_to_tensor=lambda x, dtype=None: torch.as_tensor(x, dtype=dtype),
    )
    mod = types.ModuleType("bert4keras3.backend")
    mod.ops = ops
    mod.keras = types.SimpleNamespace()
    mod.int_shape = lambda x: tuple(x.shape)
    pkg = types.ModuleType("bert4keras3")
    pkg.backend = mod
    sys.modules["bert4keras3"] = pkg
    sys.modules["bert4keras3.backend"] = mod


def demo_case(demo, name, B, T, H, N, seed, dtype, tweak=None):
    d = make_inputs(B, T, H, N, seed=seed)
    if tweak:
        tweak(d)
    tt = {n: torch.tensor(d[n], dtype=dtype, requires_grad=(n != "gy")) for n in ("r", "k", "v", "w", "u", "gy")}
    y = demo.RWKV_Kernel(B, T, H * N, H, tt["r"], tt["k"], tt["v"], tt["w"], tt["u"])
    (y * tt["gy"]).sum().backward()
    out = {n: d[n] for n in ("r", "k", "v", "w", "u", "gy")}
    def grad(n):  # autograd leaves .grad unset where y does not depend on the input (w at T=1)
        g = tt[n].grad
        return np.zeros_like(d[n], dtype=np.float64) if g is None else g.numpy()
    out.update(y=y.detach().numpy(), gr=grad("r"), gk=grad("k"), gv=grad("v"), gw=grad("w"), gu=grad("u"),
               head_size=np.int64(N))
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **out)
    print(name, {k_: getattr(v_, "shape", None) for k_, v_ in out.items()})


def ops_case(opsmod, name, B, T, H, N, seed, kinds, state_ndim4=True, explicit_map=True):
    d = make_inputs(B, T, H, N, seed=seed, with_state=True, kinds=kinds)
    init = d["init_state"] if state_ndim4 else d["init_state"][0]
    smap = d["state_map"] if explicit_map else None
    op = opsmod.RWKVKernelOperator(N, T)
    t64 = lambda a: torch.tensor(a, dtype=torch.float64)
    y, s = op(t64(d["r"]), t64(d["k"]), t64(d["v"]), t64(d["w"]), t64(d["u"]), with_state=True,
              init_state=t64(init), state_map=None if smap is None else torch.tensor(smap))
    out = {n: d[n] for n in ("r", "k", "v", "w", "u")}
    out.update(init_state=init, y=y.numpy(), s_out=s.numpy(), head_size=np.int64(N))
    if smap is not None:
        out["state_map"] = smap
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **out)
    print(name, y.shape, s.shape)


def main():
    torch.manual_seed(0)
    torch.set_num_threads(os.cpu_count() or 1)
    demo = _load(os.path.join(REF, "rwkv_v6_demo.py"), "ref_rwkv_v6_demo")
    _backend_stand_in()
    opsmod = _load(os.path.join(REF, "rwkv_kernel", "ops_rwkv_kernal.py"), "ref_ops_rwkv_kernal")

    # the reference's own CPU-runnable configuration: B2 T64 H2 N64 fp32
    demo_case(demo, "demo_cfg0_f32", 2, 64, 2, 64, seed=0, dtype=torch.float32)
    # small float64 cases pin the gradient formulas tightly
    demo_case(demo, "demo_small_f64", 2, 12, 2, 8, seed=1, dtype=torch.float64)
    demo_case(demo, "demo_t1_f64", 1, 1, 1, 8, seed=2, dtype=torch.float64)
    demo_case(demo, "demo_t3_n16_f64", 2, 3, 3, 16, seed=3, dtype=torch.float64)

    def masked(d):  # rwkv6_model.py:151 sets w = -1e9 on padded steps; also the top of the w range
        d["w"][:, 3:6, :] = -1e9
        d["w"][:, 8, :] = 1.0
    demo_case(demo, "demo_masked_f64", 2, 12, 2, 8, seed=4, dtype=torch.float64, tweak=masked)

    # state API (forward only; the reference sends no gradient through the state)
    ops_case(opsmod, "ops_state_map", 3, 10, 2, 8, seed=5, kinds=2)
    ops_case(opsmod, "ops_state_one", 3, 10, 2, 8, seed=6, kinds=1, explicit_map=False)
    ops_case(opsmod, "ops_state_perbatch", 3, 10, 2, 8, seed=7, kinds=3, explicit_map=False)
    ops_case(opsmod, "ops_state_3d", 2, 7, 2, 16, seed=8, kinds=1, state_ndim4=False, explicit_map=False)
    ops_case(opsmod, "ops_state_n64", 2, 20, 2, 64, seed=9, kinds=2)


if __name__ == "__main__":
    main()
