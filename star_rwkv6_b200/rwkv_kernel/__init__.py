"""Drop-in for the reference's ``rwkv_kernel`` package (rwkv_kernel/__init__.py:1-11): the
operator class is chosen by the KERAS_BACKEND environment variable.

    from star_rwkv6_b200.rwkv_kernel import RWKVKernelOperator
    op = RWKVKernelOperator(head_size, max_sequence_length)
    y, state = op(r, k, v, w, u, return_state=False, init_state=None, state_map=None)

``torch`` (also the default when the variable is unset) selects the PyTorch operator,
``jax`` the JAX one.  The reference's third choice, a pure keras.ops loop on whatever
device Keras runs on, is not shipped: this package has no non-CUDA path.
"""
import os

_backend = os.environ.get("KERAS_BACKEND", "torch")
if _backend == "jax":
    from .jax_rwkv_kernel import RWKVKernelOperator
elif _backend == "torch":
    from .torch_rwkv_kernel import RWKVKernelOperator
else:
    raise ImportError(
        f"KERAS_BACKEND={_backend!r}: only 'torch' and 'jax' are served by the B200 kernels; "
        "there is no framework-level fallback loop in this package")

__all__ = ["RWKVKernelOperator"]
