"""JAX ``RWKVKernelOperator`` over the library's XLA handlers.

Mirrors the reference operator (rwkv_kernel/jax_rwkv_kernel.py:31-438): the call signature
``op(r, k, v, w, u, return_state=False, init_state=None, state_map=None) -> (y, state_or_None)``, a
``jax.custom_vjp`` whose backward sums the per-batch ``gu`` (reference :163-168), the dtype policy (fp16 inputs give
fp32 outputs) and the operand orders of its three custom calls.

What differs from the reference file:
* no nvcc build at import: the handlers live in libwkv6_b200.so.  Where the library was built against jaxlib's
  ``xla/ffi/api/ffi.h`` the typed FFI handlers are used (``jax.ffi.register_ffi_target`` + ``jax.ffi.ffi_call`` with
  a ``head_size`` attribute); otherwise the legacy custom-call ABI of the reference, through ``xla._CUSTOM_CALL_TARGET``
  capsules and the 28-byte descriptor;
* the forward also returns a checkpoint buffer ([B, H, T/64, 4096] bf16), kept as a residual of the vjp beside the five
  inputs, and the backward declares a scratch result: this is what lets the op reach the chunked tensor-core kernels
  at any size (the reference's eleven-buffer backward remains available as the target ``wkv_backward``, on the
  sequential kernels);
* the reference imports ``custom_partitioning`` and never uses it; here the forward and the backward call carry a
  partitioning rule (``_jax_rules.py``): batch rows and whole heads may be sharded, time may not, ``u`` / ``gu`` follow
  the heads, and the op runs shard-locally with no collective;
* ``state_map`` must really be int64 (x64 enabled): JAX would otherwise narrow it to int32 behind the caller's back;
* states are ``S[b, h, key, value]``.

This module needs JAX with GPU support.  The containers this library was built and tested in have no JAX: the module
has never been executed there.  What is tested: the C handlers, through ctypes with the same buffer orders
(tests/test_gpu_xla_abi.py), and the framework-free rules in ``_jax_rules.py`` (tests/test_jax_rules.py).
"""
from __future__ import annotations

import ctypes
from functools import partial

import numpy as np

try:
    import jax
    import jax.numpy as jnp
except ImportError as e:  # pragma: no cover
    raise ImportError("KERAS_BACKEND=jax needs JAX installed; the B200 library itself does not") from e

from .. import _lib
from . import _jax_rules as rules

_ET = {jnp.dtype("bfloat16"): _lib.BF16, jnp.dtype("float16"): _lib.F16, jnp.dtype("float32"): _lib.F32}
_LEGACY = ("wkv_forward", "wkv_backward", "wkv_forward_with_state", "wkv_forward_ckpt", "wkv_backward_ws")
_TYPED = ("wkv6_ffi_forward", "wkv6_ffi_backward", "wkv6_ffi_forward_with_state")
_registered = None  # None = not yet, "typed" / "legacy" afterwards


def _register() -> str:
    global _registered
    if _registered:
        return _registered
    if all(hasattr(_lib.lib, s) for s in _TYPED):
        for s in _TYPED:
            jax.ffi.register_ffi_target(s, jax.ffi.pycapsule(getattr(_lib.lib, s)), platform="CUDA")
        _registered = "typed"
        return _registered
    new = ctypes.pythonapi.PyCapsule_New
    new.restype = ctypes.py_object
    new.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_void_p]
    for which, name in enumerate(_LEGACY):
        capsule = new(_lib.lib.wkv6_xla_target(which), b"xla._CUSTOM_CALL_TARGET", None)
        jax.ffi.register_ffi_target(name, capsule, platform="CUDA", api_version=0)
    _registered = "legacy"
    return _registered


def _out_dtype(dt):
    return jnp.float32 if dt == jnp.float16 else dt


def _sds(shape_dtype):
    shape, dtype = shape_dtype
    return jax.ShapeDtypeStruct(shape, jnp.dtype(dtype))


def _descriptor(r, head_size, with_state=False):
    B, T, C = r.shape
    ydt = _out_dtype(r.dtype)
    return _lib.xla_descriptor(B, T, C, C // head_size, with_state, _ET[jnp.dtype(r.dtype)], _ET[jnp.dtype(ydt)])


def _legacy(name, results, *operands, descriptor):
    return jax.ffi.ffi_call(name, results, custom_call_api_version=2, legacy_backend_config=descriptor)(*operands)


# ---- the two calls, as they run on one device (or on one shard) ---------------------------------------------------

def _fwd_local(r, k, v, w, u, head_size):
    B, T, C = r.shape
    H, name = C // head_size, jnp.dtype(r.dtype).name
    results = (jax.ShapeDtypeStruct((B, T, C), _out_dtype(r.dtype)), _sds(rules.ckpt_shape(B, T, H, head_size, name)))
    if _register() == "typed":
        return jax.ffi.ffi_call("wkv6_ffi_forward", results)(r, k, v, w, u, head_size=np.int64(head_size))
    return _legacy("wkv_forward_ckpt", results, r, k, v, w, u, descriptor=_descriptor(r, head_size))


def _bwd_local(r, k, v, w, u, gy, ckpt, head_size):
    B, T, C = r.shape
    H, name = C // head_size, jnp.dtype(r.dtype).name
    ydt = _out_dtype(r.dtype)
    g = jax.ShapeDtypeStruct((B, T, C), ydt)
    gu = jax.ShapeDtypeStruct((B,) + tuple(u.shape), ydt)
    results = (g, g, g, g, gu, _sds(rules.ws_shape(B, T, H, head_size, name)))
    if _register() == "typed":
        out = jax.ffi.ffi_call("wkv6_ffi_backward", results)(r, k, v, w, u, gy, ckpt, head_size=np.int64(head_size))
    else:
        out = _legacy("wkv_backward_ws", results, r, k, v, w, u, gy, ckpt, descriptor=_descriptor(r, head_size))
    return out[:5]


# ---- partitioning: (batch, head) pairs are independent, time is not ----------------------------------------------

def _specs(mesh, r_shape_struct, head_size):
    from jax.sharding import NamedSharding, PartitionSpec as P
    sh = r_shape_struct.sharding
    spec = tuple(sh.spec) if isinstance(sh, NamedSharding) else (None, None, None)
    x, us, bh = rules.wkv_partition_specs(spec, dict(mesh.shape), r_shape_struct.shape[2], head_size)
    ns = lambda *p: NamedSharding(mesh, P(*p))
    return ns(*x), ns(*us), bh, ns


def _make_partitioned():
    from jax.experimental.custom_partitioning import custom_partitioning

    @partial(custom_partitioning, static_argnums=(5,))
    def fwd(r, k, v, w, u, head_size):
        return _fwd_local(r, k, v, w, u, head_size)

    def fwd_infer(head_size, mesh, arg_shapes, result_shape):
        x, _, bh, ns = _specs(mesh, arg_shapes[0], head_size)
        return x, ns(*bh, None, None)

    def fwd_partition(head_size, mesh, arg_shapes, result_shape):
        x, us, bh, ns = _specs(mesh, arg_shapes[0], head_size)
        return mesh, lambda r, k, v, w, u: _fwd_local(r, k, v, w, u, head_size), (x, ns(*bh, None, None)), (x, x, x, x, us)

    fwd.def_partition(infer_sharding_from_operands=fwd_infer, partition=fwd_partition,
                      sharding_rule="b t c, b t c, b t c, b t c, h n -> b t c, b h q z")

    @partial(custom_partitioning, static_argnums=(7,))
    def bwd(r, k, v, w, u, gy, ckpt, head_size):
        return _bwd_local(r, k, v, w, u, gy, ckpt, head_size)

    def bwd_infer(head_size, mesh, arg_shapes, result_shape):
        x, _, bh, ns = _specs(mesh, arg_shapes[0], head_size)
        return x, x, x, x, ns(*bh, None)

    def bwd_partition(head_size, mesh, arg_shapes, result_shape):
        x, us, bh, ns = _specs(mesh, arg_shapes[0], head_size)
        return (mesh, lambda r, k, v, w, u, gy, ckpt: _bwd_local(r, k, v, w, u, gy, ckpt, head_size),
                (x, x, x, x, ns(*bh, None)), (x, x, x, x, us, x, ns(*bh, None, None)))

    bwd.def_partition(infer_sharding_from_operands=bwd_infer, partition=bwd_partition,
                      sharding_rule="b t c, b t c, b t c, b t c, h n, b t c, b h q z -> b t c, b t c, b t c, b t c, b h n")
    return fwd, bwd


_partitioned = None


def _calls():
    global _partitioned
    if _partitioned is None:
        _partitioned = _make_partitioned()
    return _partitioned


@partial(jax.custom_vjp, nondiff_argnums=(5,))
def wkv(r, k, v, w, u, head_size):
    return _calls()[0](r, k, v, w, u, head_size)[0]


def _wkv_fwd(r, k, v, w, u, head_size):
    y, ckpt = _calls()[0](r, k, v, w, u, head_size)
    return y, (r, k, v, w, u, ckpt)


def _wkv_bwd(head_size, res, gy):
    r, k, v, w, u, ckpt = res
    gr, gk, gv, gw, gu = _calls()[1](r, k, v, w, u, gy.astype(_out_dtype(r.dtype)), ckpt, head_size)
    cast = lambda g: g.astype(r.dtype)
    return cast(gr), cast(gk), cast(gv), cast(gw), jnp.sum(gu, 0).astype(u.dtype)


wkv.defvjp(_wkv_fwd, _wkv_bwd)


class RWKVKernelOperator:
    def __init__(self, head_size, max_sequence_length=None):
        self.head_size = int(head_size)
        self.max_sequence_length = max_sequence_length  # advisory: T is a run-time value
        _register()

    def __call__(self, r, k, v, w, u, return_state=False, init_state=None, state_map=None):
        B, T, C = r.shape
        assert C % self.head_size == 0
        H, N = C // self.head_size, self.head_size
        assert r.dtype == k.dtype == v.dtype == w.dtype == u.dtype
        assert jnp.dtype(r.dtype) in _ET
        u = jnp.reshape(u, (H, N))
        if not return_state:
            assert init_state is None and state_map is None, "init_state / state_map need return_state=True"
            return wkv(r, k, v, w, u, N), None
        ydt = _out_dtype(r.dtype)
        has = init_state is not None
        if has:
            if init_state.ndim == 3:
                init_state = init_state[None]
            assert init_state.shape[1:] == (H, N, N) and init_state.shape[0] <= B
            assert init_state.dtype == ydt, f"init_state must be {ydt}"
            kinds = init_state.shape[0]
            if state_map is None:
                assert kinds in (1, B), "state_map cannot be inferred; pass it explicitly"
                state_map = np.zeros((B,), np.int64) if kinds == 1 else np.arange(B, dtype=np.int64)
            state_map = jnp.asarray(state_map)
            if state_map.dtype == jnp.int32 and jax.config.jax_enable_x64:
                state_map = state_map.astype(jnp.int64)
            rules.check_state_map_dtype(jnp.dtype(state_map.dtype).name)
            assert state_map.shape == (B,)
        else:
            assert state_map is None, "state_map needs an init_state"
        results = (jax.ShapeDtypeStruct((B, T, C), ydt), jax.ShapeDtypeStruct((B, H, N, N), ydt))
        if _register() == "typed":
            s = init_state if has else jnp.zeros((1, H, N, N), ydt)
            m = state_map if has else jnp.zeros((B,), jnp.int32)
            return jax.ffi.ffi_call("wkv6_ffi_forward_with_state", results)(r, k, v, w, u, s, m, head_size=np.int64(N),
                                                                              has_state=np.bool_(has))
        desc = _descriptor(r, N, with_state=has)
        ops = (state_map, r, k, v, w, u, init_state) if has else (r, k, v, w, u)
        y, s = _legacy("wkv_forward_with_state", results, *ops, descriptor=desc)
        return y, s
