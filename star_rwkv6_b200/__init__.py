"""B200-native (sm_100a) RWKV-6 WKV recurrence, a drop-in behind the operator surfaces of
infiy-quine/STAR-RWKV6.  The CUDA library (libwkv6_b200.so, C ABI in include/wkv6_b200.h)
is mandatory; importing this package without it raises."""
from . import _lib  # noqa: F401  (loads the shared library or raises)
from ._lib import VARIANT_AUTO, VARIANT_CHUNK, VARIANT_SEQ, WKV6Error
from .ops import backward_raw, forward_raw, wkv6, wkv6_with_state

__all__ = ["wkv6", "wkv6_with_state", "forward_raw", "backward_raw", "WKV6Error",
           "VARIANT_AUTO", "VARIANT_SEQ", "VARIANT_CHUNK"]
