"""ctypes binding of oracle/_ref/libref_wkv6_cuda.so: the reference's own CUDA kernels (rwkv_kernel/jax_kernel/
rwkv_kernels.cu, compiled unchanged for sm_100a by oracle/build_ref_cuda.py), driven with torch device buffers in the
reference's buffer orders.  Test / benchmark infrastructure only; the product never imports this module."""
import ctypes
import os
import struct

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "_ref", "libref_wkv6_cuda.so")
HEAD_SIZE, MAX_T = 64, 4096          # the -D_N_ / -D_T_ the library was compiled with
_CODES = {"bfloat16": 0, "float16": 1, "float32": 2}
_lib = None


def available() -> bool:
    return os.path.exists(LIB)


def lib():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(LIB)
        for f in (_lib.ref_wkv6_forward, _lib.ref_wkv6_backward):
            f.restype = None
            f.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_void_p), ctypes.c_char_p, ctypes.c_size_t]
        _lib.ref_wkv6_last_cuda_error.restype = ctypes.c_int
    return _lib


def descriptor(B, T, C, H, x_dtype: str, y_dtype: str) -> bytes:
    """The reference's WKVDescriptor (kernels.h:32-42): int B, T, C, H; bool S; enum x_type, y_type; 28 bytes."""
    return struct.pack("<iiii?3xii", B, T, C, H, False, _CODES[x_dtype], _CODES[y_dtype])


def _bufs(tensors):
    return (ctypes.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])


def forward(r, k, v, w, u, y, stream):
    """Enqueue the reference forward on ``stream``: buffers [r, k, v, w, u, y] (rwkv_kernels.cu:451-464)."""
    B, T, C = r.shape
    assert C % HEAD_SIZE == 0 and T <= MAX_T
    name = str(r.dtype).split(".")[-1]
    d = descriptor(B, T, C, C // HEAD_SIZE, name, str(y.dtype).split(".")[-1])
    lib().ref_wkv6_forward(ctypes.c_void_p(stream), _bufs([r, k, v, w, u, y]), d, len(d))


def backward(r, k, v, w, u, gy, gr, gk, gv, gw, gu, stream):
    """Enqueue the reference backward (four kernels): buffers [r, k, v, w, u, gy, gr, gk, gv, gw, gu], gu is [B, C]
    (rwkv_kernels.cu:493-508)."""
    B, T, C = r.shape
    assert C % HEAD_SIZE == 0 and 3 <= T <= MAX_T
    name = str(r.dtype).split(".")[-1]
    d = descriptor(B, T, C, C // HEAD_SIZE, name, str(gy.dtype).split(".")[-1])
    lib().ref_wkv6_backward(ctypes.c_void_p(stream), _bufs([r, k, v, w, u, gy, gr, gk, gv, gw, gu]), d, len(d))
