"""JAX ``RWKVKernelOperator`` over the library's XLA legacy custom-call handlers.

Mirrors the reference operator (rwkv_kernel/jax_rwkv_kernel.py:31-438): three custom calls named
``wkv_forward`` / ``wkv_backward`` / ``wkv_forward_with_state`` with the reference's operand orders and 28-byte
opaque descriptor, a ``jax.custom_vjp`` whose residuals are the five inputs and whose backward sums the per-batch
``gu`` (reference :163-168), and the call signature
``op(r, k, v, w, u, return_state=False, init_state=None, state_map=None) -> (y, state_or_None)``.

What differs from the reference file:
* no nvcc build at import: the handlers live in libwkv6_b200.so and are wrapped in ``xla._CUSTOM_CALL_TARGET``
  capsules here; registration and lowering go through ``jax.ffi`` (``register_ffi_target(api_version=0)``,
  ``ffi_call(custom_call_api_version=2, legacy_backend_config=descriptor)``) instead of the jaxlib internals
  the reference used, which current JAX no longer has;
* the reference imports ``custom_partitioning`` and never uses it; here ``wkv`` is wrapped so that the batch
  dimension and the head dimension (multiples of head_size on the channel axis) may be sharded and the op runs
  shard-locally with no collective; T must stay unsharded;
* states are ``S[b, h, key, value]``.

This module needs JAX with GPU support.  It is not exercised by the test-suite of this repository (the build
containers have no JAX); the C handlers it calls are tested through ctypes in tests/test_gpu_xla_abi.py.
"""
from __future__ import annotations

import ctypes
from functools import partial

try:
    import jax
    import jax.numpy as jnp
except ImportError as e:  # pragma: no cover
    raise ImportError("KERAS_BACKEND=jax needs JAX installed; the B200 library itself does not") from e

from .. import _lib

_ET = {jnp.dtype("bfloat16"): _lib.BF16, jnp.dtype("float16"): _lib.F16, jnp.dtype("float32"): _lib.F32}
_TARGETS = ("wkv_forward", "wkv_backward", "wkv_forward_with_state")
_registered = False


def _register():
    global _registered
    if _registered:
        return
    new = ctypes.pythonapi.PyCapsule_New
    new.restype = ctypes.py_object
    new.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_void_p]
    for which, name in enumerate(_TARGETS):
        capsule = new(_lib.lib.wkv6_xla_target(which), b"xla._CUSTOM_CALL_TARGET", None)
        jax.ffi.register_ffi_target(name, capsule, platform="CUDA", api_version=0)
    _registered = True


def _out_dtype(dt):
    return jnp.float32 if dt == jnp.float16 else dt


def _call(name, results, *operands, descriptor):
    return jax.ffi.ffi_call(name, results, custom_call_api_version=2, legacy_backend_config=descriptor)(*operands)


def _fwd_call(r, k, v, w, u, head_size):
    B, T, C = r.shape
    ydt = _out_dtype(r.dtype)
    desc = _lib.xla_descriptor(B, T, C, C // head_size, False, _ET[jnp.dtype(r.dtype)], _ET[jnp.dtype(ydt)])
    return _call("wkv_forward", jax.ShapeDtypeStruct((B, T, C), ydt), r, k, v, w, u, descriptor=desc)


def _bwd_call(r, k, v, w, u, gy, head_size):
    B, T, C = r.shape
    ydt = _out_dtype(r.dtype)
    desc = _lib.xla_descriptor(B, T, C, C // head_size, False, _ET[jnp.dtype(r.dtype)], _ET[jnp.dtype(ydt)])
    g = jax.ShapeDtypeStruct((B, T, C), ydt)
    gu = jax.ShapeDtypeStruct((B,) + tuple(u.shape), ydt)
    return _call("wkv_backward", (g, g, g, g, gu), r, k, v, w, u, gy, descriptor=desc)


@partial(jax.custom_vjp, nondiff_argnums=(5,))
def wkv(r, k, v, w, u, head_size):
    return _fwd_call(r, k, v, w, u, head_size)


def _wkv_fwd(r, k, v, w, u, head_size):
    return _fwd_call(r, k, v, w, u, head_size), (r, k, v, w, u)


def _wkv_bwd(head_size, res, gy):
    r, k, v, w, u = res
    gr, gk, gv, gw, gu = _bwd_call(r, k, v, w, u, gy.astype(_out_dtype(r.dtype)), head_size)
    cast = lambda g: g.astype(r.dtype)
    return cast(gr), cast(gk), cast(gv), cast(gw), jnp.sum(gu, 0).astype(u.dtype)


wkv.defvjp(_wkv_fwd, _wkv_bwd)


def sharded_wkv(mesh, batch_axis=None, head_axis=None):
    """wkv under a mesh: batch rows over ``batch_axis`` and heads over ``head_axis``, shard-local, no collective.
    (b, h) pairs are independent, so each device runs the op on its [B/db, T, C/dh] block with its [H/dh, N] slice
    of u; gu comes back per batch row and its batch sum is an ordinary psum-free jnp.sum over the sharded axis."""
    from jax.experimental.shard_map import shard_map
    from jax.sharding import PartitionSpec as P

    x = P(batch_axis, None, head_axis)
    us = P(head_axis, None)

    def build(head_size):
        return shard_map(lambda r, k, v, w, u: wkv(r, k, v, w, u, head_size), mesh=mesh,
                         in_specs=(x, x, x, x, us), out_specs=x, check_rep=False)
    return build


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
                state_map = jnp.zeros((B,), jnp.int64) if kinds == 1 else jnp.arange(B, dtype=jnp.int64)
            state_map = jnp.asarray(state_map, dtype=jnp.int64)
            assert state_map.shape == (B,)
        else:
            assert state_map is None, "state_map needs an init_state"
        desc = _lib.xla_descriptor(B, T, C, H, has, _ET[jnp.dtype(r.dtype)], _ET[jnp.dtype(ydt)])
        results = (jax.ShapeDtypeStruct((B, T, C), ydt), jax.ShapeDtypeStruct((B, H, N, N), ydt))
        ops = (state_map, r, k, v, w, u, init_state) if has else (r, k, v, w, u)
        y, s = _call("wkv_forward_with_state", results, *ops, descriptor=desc)
        return y, s
