"""The JAX operator module (star_rwkv6_b200/rwkv_kernel/jax_rwkv_kernel.py) driven through a stand-in for JAX.

JAX is not installed where this library is developed, so the module cannot run for real.  This test gives it a small
numpy-backed stand-in with exactly the entry points the module uses (jax.ffi.register_ffi_target / pycapsule / ffi_call,
jax.ShapeDtypeStruct, jax.custom_vjp, jax.config, jax.numpy basics, custom_partitioning, NamedSharding / PartitionSpec) and
checks what the module asks of JAX: which targets it registers and how, which call it lowers to, the operand order, the
declared result shapes and dtypes (including the two extra buffers of the chunked kernels), the 28-byte descriptor, the
dtype policy, the gu reduction over batch rows, the int64 rule for state_map, and the partitioning rule.  It does not prove
that real JAX accepts these calls - only that the module is importable, consistent with the C ABI's buffer orders
(tests/test_gpu_xla_abi.py drives those on a GPU) and does what its docstring says.
"""
import importlib
import sys
import types

import numpy as np
import pytest


class _BF16:
    name = "bfloat16"

    def __repr__(self):
        return "bfloat16"


_BF = _BF16()


def _dtype(x):
    if x is _BF or x == "bfloat16":
        return _BF
    return np.dtype(x)


class _SDS:
    def __init__(self, shape, dtype):
        self.shape, self.dtype, self.sharding = tuple(shape), dtype, None


class _Log:
    def __init__(self):
        self.registered, self.calls = [], []


def _fake_jax(log):
    jax = types.ModuleType("jax")
    jnp = types.ModuleType("jax.numpy")
    jnp.dtype = _dtype
    jnp.float16, jnp.float32, jnp.int32, jnp.int64 = np.float16, np.float32, np.int32, np.int64
    jnp.reshape, jnp.asarray, jnp.zeros, jnp.sum = np.reshape, np.asarray, np.zeros, np.sum
    jax.numpy = jnp
    jax.ShapeDtypeStruct = _SDS
    jax.config = types.SimpleNamespace(jax_enable_x64=False)

    ffi = types.ModuleType("jax.ffi")
    ffi.pycapsule = lambda fn: ("capsule", fn)
    ffi.register_ffi_target = lambda name, capsule, **kw: log.registered.append((name, capsule, kw))
    ffi.include_dir = lambda: "/nonexistent"

    def ffi_call(name, results, **kw):
        def run(*operands, **attrs):
            log.calls.append(dict(name=name, results=results, kw=kw, operands=operands, attrs=attrs))
            mk = lambda s: np.ones(s.shape, dtype=np.float32 if s.dtype is _BF else s.dtype)
            return tuple(mk(s) for s in results)
        return run
    ffi.ffi_call = ffi_call
    jax.ffi = ffi

    class custom_vjp:
        def __init__(self, fn, nondiff_argnums=()):
            self.fn, self.nondiff_argnums = fn, nondiff_argnums

        def __call__(self, *a):
            return self.fn(*a)

        def defvjp(self, fwd, bwd):
            self.fwd, self.bwd = fwd, bwd
    jax.custom_vjp = custom_vjp

    exp = types.ModuleType("jax.experimental")
    cp = types.ModuleType("jax.experimental.custom_partitioning")

    class custom_partitioning:
        def __init__(self, fn, static_argnums=()):
            self.fn, self.static_argnums, self.rules = fn, static_argnums, None

        def __call__(self, *a):
            return self.fn(*a)

        def def_partition(self, **kw):
            self.rules = kw
    cp.custom_partitioning = custom_partitioning
    exp.custom_partitioning = cp
    jax.experimental = exp

    sh = types.ModuleType("jax.sharding")

    class PartitionSpec(tuple):
        def __new__(cls, *p):
            return super().__new__(cls, p)

    class NamedSharding:
        def __init__(self, mesh, spec):
            self.mesh, self.spec = mesh, spec
    sh.PartitionSpec, sh.NamedSharding = PartitionSpec, NamedSharding
    jax.sharding = sh
    return {"jax": jax, "jax.numpy": jnp, "jax.ffi": ffi, "jax.experimental": exp,
            "jax.experimental.custom_partitioning": cp, "jax.sharding": sh}


@pytest.fixture()
def mod():
    log = _Log()
    fakes = _fake_jax(log)
    saved = {k: sys.modules.get(k) for k in fakes}
    sys.modules.update(fakes)
    sys.modules.pop("star_rwkv6_b200.rwkv_kernel.jax_rwkv_kernel", None)
    try:
        m = importlib.import_module("star_rwkv6_b200.rwkv_kernel.jax_rwkv_kernel")
        yield m, log
    finally:
        sys.modules.pop("star_rwkv6_b200.rwkv_kernel.jax_rwkv_kernel", None)
        for k, v in saved.items():
            if v is None:
                sys.modules.pop(k, None)
            else:
                sys.modules[k] = v


def _inputs(B, T, H, N, dtype):
    rng = np.random.default_rng(0)
    mk = lambda: rng.standard_normal((B, T, H * N)).astype(dtype)
    return mk(), mk(), mk(), mk(), rng.standard_normal((H * N,)).astype(dtype)


def test_registration_and_forward_lowering(mod):
    m, log = mod
    from star_rwkv6_b200 import _lib
    from star_rwkv6_b200.rwkv_kernel import _jax_rules as R
    B, T, H, N = 2, 100, 2, 64
    op = m.RWKVKernelOperator(N, T)
    # no typed handlers in a library built without jaxlib's headers: the five legacy targets, api_version 0, as capsules
    assert [r[0] for r in log.registered] == ["wkv_forward", "wkv_backward", "wkv_forward_with_state", "wkv_forward_ckpt",
                                              "wkv_backward_ws"]
    assert all(r[2] == dict(platform="CUDA", api_version=0) for r in log.registered)
    assert all(type(r[1]).__name__ == "PyCapsule" for r in log.registered)
    r, k, v, w, u = _inputs(B, T, H, N, np.float32)
    y, none = op(r, k, v, w, u)
    assert none is None and y.shape == (B, T, H * N)
    c = log.calls[-1]
    assert c["name"] == "wkv_forward_ckpt" and c["kw"]["custom_call_api_version"] == 2
    assert c["kw"]["legacy_backend_config"] == _lib.xla_descriptor(B, T, H * N, H, False, _lib.F32, _lib.F32)
    assert len(c["kw"]["legacy_backend_config"]) == 28
    assert [o.shape for o in c["operands"]] == [(B, T, H * N)] * 4 + [(H, N)]          # u arrives as [H, N]
    assert c["operands"][0] is r and c["operands"][3] is w
    ysd, cksd = c["results"]
    assert ysd.shape == (B, T, H * N) and ysd.dtype == np.float32
    assert (cksd.shape, getattr(cksd.dtype, "name", None)) == R.ckpt_shape(B, T, H, N, "float32")


def test_backward_lowering_and_gu_reduction(mod):
    m, log = mod
    from star_rwkv6_b200.rwkv_kernel import _jax_rules as R
    B, T, H, N = 3, 64, 2, 64
    m.RWKVKernelOperator(N, T)
    r, k, v, w, u = _inputs(B, T, H, N, np.float16)
    u = u.reshape(H, N)
    y, res = m.wkv.fwd(r, k, v, w, u, N)
    assert y.dtype == np.float32                                  # fp16 inputs give fp32 outputs (the reference's policy)
    assert len(res) == 6 and res[5].shape == R.ckpt_shape(B, T, H, N, "float16")[0]   # the checkpoint buffer is a residual
    gy = np.ones((B, T, H * N), np.float16)
    grads = m.wkv.bwd(N, res, gy)
    c = log.calls[-1]
    assert c["name"] == "wkv_backward_ws"
    assert [o.shape for o in c["operands"]] == [(B, T, H * N)] * 4 + [(H, N), (B, T, H * N), res[5].shape]
    assert c["operands"][5].dtype == np.float32                   # gy is cast to the output dtype before the call
    shapes = [s.shape for s in c["results"]]
    assert shapes[:5] == [(B, T, H * N)] * 4 + [(B, H, N)] and shapes[5] == R.ws_shape(B, T, H, N, "float16")[0]
    assert [g.shape for g in grads] == [(B, T, H * N)] * 4 + [(H, N)]
    assert all(g.dtype == np.float16 for g in grads[:4]) and grads[4].dtype == np.float16
    assert np.all(grads[4] == B)                                  # the stand-in returns ones: the batch rows were summed


def test_state_api_and_state_map_rule(mod):
    m, log = mod
    B, T, H, N = 4, 32, 2, 64
    op = m.RWKVKernelOperator(N, T)
    r, k, v, w, u = _inputs(B, T, H, N, np.float32)
    y, s = op(r, k, v, w, u, return_state=True)
    c = log.calls[-1]
    assert c["name"] == "wkv_forward_with_state" and len(c["operands"]) == 5          # S = 0: [r, k, v, w, u, y, ys]
    assert [x.shape for x in c["results"]] == [(B, T, H * N), (B, H, N, N)]
    init = np.zeros((1, H, N, N), np.float32)
    op(r, k, v, w, u, return_state=True, init_state=init)
    c = log.calls[-1]
    assert len(c["operands"]) == 7 and c["operands"][0].dtype == np.int64 and c["operands"][0].shape == (B,)   # map first
    assert c["operands"][6] is init
    with pytest.raises(TypeError):                                                       # int32 map without x64: refused
        op(r, k, v, w, u, return_state=True, init_state=init, state_map=np.zeros((B,), np.int32))
    with pytest.raises(AssertionError):
        op(r, k, v, w, u, init_state=init)                                               # needs return_state=True


def test_partitioning_rule(mod):
    m, log = mod
    fwd, bwd = m._calls()
    assert fwd.static_argnums == (5,) and bwd.static_argnums == (7,)
    assert fwd.rules["sharding_rule"] == "b t c, b t c, b t c, b t c, h n -> b t c, b h q z"
    from jax.sharding import NamedSharding, PartitionSpec as P
    mesh = types.SimpleNamespace(shape={"data": 2, "model": 4})
    arg = _SDS((8, 128, 2048), np.float32)
    arg.sharding = NamedSharding(mesh, P("data", None, "model"))
    y_sh, ck_sh = fwd.rules["infer_sharding_from_operands"](64, mesh, [arg] * 5, None)
    assert tuple(y_sh.spec) == ("data", None, "model")            # batch and channel (whole heads) split, time never
    assert tuple(ck_sh.spec)[:2] == ("data", "model")
    arg.sharding = NamedSharding(mesh, P(None, "data", None))    # a split along time is taken back: T is sequential
    y_sh, _ = fwd.rules["infer_sharding_from_operands"](64, mesh, [arg] * 5, None)
    assert tuple(y_sh.spec)[1] is None
