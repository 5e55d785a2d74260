"""ctypes front end of the C oracle (oracle/wkv6_oracle.c).  Test infrastructure only.

``fwd`` / ``bwd`` take numpy arrays shaped like the operator's tensors and run
the float64 (default) or float32 instantiation on all host threads.
"""
from __future__ import annotations

import ctypes
import os

import numpy as np

from . import build_oracle
from .wkv6_oracle import resolve_state

_lib = None


def lib():
    global _lib
    if _lib is None:
        path = build_oracle.LIB
        if not os.path.exists(path):
            path = build_oracle.build()
        _lib = ctypes.CDLL(path)
    return _lib


def threads() -> int:
    return int(lib().wkv6_oracle_threads_f64())


def use_all_cores() -> int:
    """Run on every core this process may use, whatever OMP_NUM_THREADS says (torchrun sets it to 1 for its
    workers).  Returns the thread count now in force."""
    import os
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    lib().wkv6_oracle_set_threads_f64(n)
    return threads()


def _prep(x, dt):
    return np.ascontiguousarray(np.asarray(x, dtype=dt))


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p) if a is not None else None


def fwd(r, k, v, w, u, head_size, init_state=None, state_map=None, dtype=np.float64):
    sfx = "f64" if dtype == np.float64 else "f32"
    r, k, v, w = (_prep(x, dtype) for x in (r, k, v, w))
    B, T, C = r.shape
    N = head_size
    H = C // N
    u = _prep(u, dtype).reshape(H, N)
    s_in = None
    if init_state is not None:
        s_in = _prep(resolve_state(B, H, N, init_state, state_map), dtype)
    y = np.empty_like(r)
    s_out = np.empty((B, H, N, N), dtype=dtype)
    fn = getattr(lib(), f"wkv6_oracle_fwd_{sfx}")
    fn(B, T, H, N, _p(r), _p(k), _p(v), _p(w), _p(u), _p(s_in), _p(y), _p(s_out))
    return y, s_out


def bwd(r, k, v, w, u, gy, head_size, init_state=None, state_map=None, dtype=np.float64):
    sfx = "f64" if dtype == np.float64 else "f32"
    r, k, v, w, gy = (_prep(x, dtype) for x in (r, k, v, w, gy))
    B, T, C = r.shape
    N = head_size
    H = C // N
    u = _prep(u, dtype).reshape(H, N)
    s_in = None
    if init_state is not None:
        s_in = _prep(resolve_state(B, H, N, init_state, state_map), dtype)
    gr, gk, gv, gw = (np.empty_like(r) for _ in range(4))
    gu = np.empty((B, H, N), dtype=dtype)
    fn = getattr(lib(), f"wkv6_oracle_bwd_{sfx}")
    fn(B, T, H, N, _p(r), _p(k), _p(v), _p(w), _p(u), _p(gy), _p(s_in),
       _p(gr), _p(gk), _p(gv), _p(gw), _p(gu))
    return gr, gk, gv, gw, gu
