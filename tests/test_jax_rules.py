"""The framework-free rules of the JAX operator (shapes of the extra buffers, state-map dtype, partitioning)."""
import ctypes

import pytest

from star_rwkv6_b200 import _lib as L
from star_rwkv6_b200.rwkv_kernel import _jax_rules as R


def _bytes(shape_dtype):
    shape, dtype = shape_dtype
    n = {"bfloat16": 2, "int32": 4, "float32": 4}[dtype]
    for s in shape:
        n *= s
    return n


@pytest.mark.parametrize("B,T,H,N,name,code", [(8, 4096, 32, 64, "bfloat16", 0), (2, 100, 3, 64, "bfloat16", 0), (1, 1, 1, 64, "bfloat16", 0),
                                                (2, 64, 2, 64, "float32", 2), (2, 64, 4, 32, "bfloat16", 0), (3, 50, 2, 16, "float16", 1)])
def test_extra_buffers_are_large_enough(B, T, H, N, name, code):
    """The shapes the JAX side declares cover what the library asks for the same problem."""
    y_code = 2 if code == 1 else code
    desc = L.xla_descriptor(B, T, H * N, H, False, code, y_code)
    need_ck, need_ws = (L.lib.wkv6_xla_buffer_bytes(desc, len(desc), i) for i in (0, 1))
    assert _bytes(R.ckpt_shape(B, T, H, N, name)) >= need_ck
    assert _bytes(R.ws_shape(B, T, H, N, name)) >= need_ws
    # and both split with the (batch, head) pairs
    assert R.ckpt_shape(B, T, H, N, name)[0][:2] == (B, H) and R.ws_shape(B, T, H, N, name)[0][:2] == (B, H)


def test_state_map_must_be_int64():
    R.check_state_map_dtype("int64")
    with pytest.raises(TypeError, match="jax_enable_x64"):
        R.check_state_map_dtype("int32")


def test_partitioning_rule():
    mesh = {"data": 4, "model": 2, "seq": 2}
    # batch over data, heads over model: kept; u and the (batch, head) buffers follow
    x, u, bh = R.wkv_partition_specs(("data", None, "model"), mesh, C=2048, head_size=64)
    assert x == ("data", None, "model") and u == ("model", None) and bh == ("data", "model")
    # a sharded time axis is replaced by a replicated one
    x, u, bh = R.wkv_partition_specs(("data", "seq", None), mesh, C=2048, head_size=64)
    assert x == ("data", None, None) and u == (None, None) and bh == ("data", None)
    # a channel split that would cut through a head is dropped (3 heads over 2 devices)
    x, u, bh = R.wkv_partition_specs((None, None, "model"), mesh, C=192, head_size=64)
    assert x == (None, None, None) and u == (None, None)
    # several mesh axes on one dimension
    x, u, bh = R.wkv_partition_specs((("data", "seq"), None, "model"), mesh, C=2048, head_size=64)
    assert x == (("data", "seq"), None, "model") and bh == (("data", "seq"), "model")
    # short specs are padded
    assert R.wkv_partition_specs(("data",), mesh, C=128, head_size=64)[0] == ("data", None, None)
