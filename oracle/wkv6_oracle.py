"""CPU oracle for the RWKV-6 WKV recurrence (forward, state API, backward).

TEST INFRASTRUCTURE ONLY.  Nothing under ``oracle/`` is part of the shipped
product path: only the test-suite, the smoke check and the CPU-baseline /
reference leg of the benchmark may import it, and only as the checker.

This is a float64 numpy restatement of the reference's non-CUDA operator:

* forward recurrence and ``init_state`` / ``state_map`` / returned state:
  ``rwkv_kernel/ops_rwkv_kernal.py:28-97`` (loop at :83-95); the same loop
  with a zero initial state is ``rwkv_v6_demo.py:10-43``.
* backward: the reference obtains gradients by autograd through that loop
  (``deprecated_code/wkv_torch.py:56``); its CUDA kernels state the closed
  forms (``rwkv_kernel/jax_kernel/rwkv_kernels.cu:205-407``).  Here the
  closed forms are evaluated with an explicit reverse-time loop.

Parity pin: ``tests/golden/*.npz`` were produced by running the reference's
own Python (``rwkv_v6_demo.RWKV_Kernel`` with torch autograd, and
``ops_rwkv_kernal.RWKVKernelOperator`` over a torch-backed stand-in for its
``bert4keras3.backend`` import) by ``tests/golden/make_golden.py``; the
CPU test tier checks this oracle against every one of them.

Conventions (all arrays C-contiguous):
  r, k, v, w : [B, T, C], C = H*N, channel c = h*N + i
  u          : [H, N] (any shape with H*N elements)
  state      : S[b, h, key i, value j]   (the layout of ops_rwkv_kernal.py:85-91)
  y_t[j]   = sum_i r_t[i] * (u[i] k_t[i] v_t[j] + S_{t-1}[i, j])
  S_t[i,j] = exp(-exp(w_t[i])) * S_{t-1}[i, j] + k_t[i] v_t[j]
"""
from __future__ import annotations

import numpy as np


def resolve_state(B, H, N, init_state, state_map):
    """Initial state per batch row, following ops_rwkv_kernal.py:41-72.

    Returns float64 [B, H, N, N].  Raises AssertionError / ValueError on the
    same conditions as the reference.
    """
    if init_state is None:
        assert state_map is None
        return np.zeros((B, H, N, N), dtype=np.float64)
    init_state = np.asarray(init_state, dtype=np.float64)
    assert init_state.ndim in (3, 4)
    if init_state.ndim == 3:
        assert init_state.shape == (H, N, N)
        init_state = init_state[None]
    else:
        assert init_state.shape[1:] == (H, N, N)
        assert init_state.shape[0] <= B
    kinds = init_state.shape[0]
    if state_map is None:
        if kinds == 1:
            state_map = np.zeros((B,), dtype=np.int64)
        elif kinds == B:
            state_map = np.arange(B, dtype=np.int64)
        else:
            raise ValueError("state_map cannot be inferred; pass it explicitly")
    else:
        state_map = np.asarray(state_map)
        assert state_map.dtype in (np.int32, np.int64)
        state_map = state_map.astype(np.int64)
        assert state_map.shape == (B,)
        assert (state_map >= 0).all() and (state_map < kinds).all()
    return init_state[state_map]


def wkv6_forward(r, k, v, w, u, head_size, init_state=None, state_map=None):
    """Forward pass.  Returns (y [B,T,C], final state [B,H,N,N]) in float64."""
    r = np.asarray(r, dtype=np.float64)
    k = np.asarray(k, dtype=np.float64)
    v = np.asarray(v, dtype=np.float64)
    w = np.asarray(w, dtype=np.float64)
    B, T, C = r.shape
    N = head_size
    assert C % N == 0
    H = C // N
    u = np.asarray(u, dtype=np.float64).reshape(H, N)
    r4 = r.reshape(B, T, H, N)
    k4 = k.reshape(B, T, H, N)
    v4 = v.reshape(B, T, H, N)
    d4 = np.exp(-np.exp(w.reshape(B, T, H, N)))
    S = resolve_state(B, H, N, init_state, state_map).copy()
    y = np.empty((B, T, H, N), dtype=np.float64)
    for t in range(T):
        kv = k4[:, t, :, :, None] * v4[:, t, :, None, :]          # [B,H,i,j]
        y[:, t] = np.einsum("bhi,bhij->bhj", r4[:, t], u[None, :, :, None] * kv + S)
        S = d4[:, t, :, :, None] * S + kv
    return y.reshape(B, T, C), S


def wkv6_backward(r, k, v, w, u, gy, head_size, init_state=None, state_map=None):
    """Gradients of sum(y * gy) w.r.t. r, k, v, w and u.

    No gradient flows through the returned state (as in the reference:
    rwkv_kernels.cu:252-338 start the reverse state at zero).  ``gu`` is
    returned per batch row, [B, H, N], like the reference kernels
    (rwkv_kernels.cu:243-249); the batch sum happens in the caller
    (jax_rwkv_kernel.py:166, torch_rwkv_kernel.py:73).
    """
    r = np.asarray(r, dtype=np.float64)
    k = np.asarray(k, dtype=np.float64)
    v = np.asarray(v, dtype=np.float64)
    w = np.asarray(w, dtype=np.float64)
    gy = np.asarray(gy, dtype=np.float64)
    B, T, C = r.shape
    N = head_size
    H = C // N
    u = np.asarray(u, dtype=np.float64).reshape(H, N)
    r4 = r.reshape(B, T, H, N)
    k4 = k.reshape(B, T, H, N)
    v4 = v.reshape(B, T, H, N)
    g4 = gy.reshape(B, T, H, N)
    ew = np.exp(w.reshape(B, T, H, N))
    d4 = np.exp(-ew)

    # forward sweep: gr, gu need S_{t-1}; keep every S_{t-1} for the gw term
    S = resolve_state(B, H, N, init_state, state_map).copy()
    S_prev = np.empty((T, B, H, N, N), dtype=np.float64)
    gr = np.empty_like(r4)
    gu = np.zeros((B, H, N), dtype=np.float64)
    for t in range(T):
        S_prev[t] = S
        vg = np.einsum("bhj,bhj->bh", v4[:, t], g4[:, t])            # v_t . gy_t
        gr[:, t] = u[None] * k4[:, t] * vg[..., None] + np.einsum("bhij,bhj->bhi", S, g4[:, t])
        gu += r4[:, t] * k4[:, t] * vg[..., None]
        S = d4[:, t, :, :, None] * S + k4[:, t, :, :, None] * v4[:, t, :, None, :]

    # reverse sweep: A_t = sum_{tau>t} (prod_{t<s<tau} d_s) r_tau (x) gy_tau
    A = np.zeros((B, H, N, N), dtype=np.float64)
    gk = np.empty_like(r4)
    gv = np.empty_like(r4)
    gw = np.empty_like(r4)
    for t in range(T - 1, -1, -1):
        ur = u[None] * r4[:, t]                                        # [B,H,i]
        M = ur[..., None] * g4[:, t, :, None, :] + A                   # [B,H,i,j]
        gk[:, t] = np.einsum("bhij,bhj->bhi", M, v4[:, t])
        gv[:, t] = np.einsum("bhij,bhi->bhj", M, k4[:, t])
        gw[:, t] = -ew[:, t] * d4[:, t] * np.einsum("bhij,bhij->bhi", S_prev[t], A)
        A = r4[:, t, :, :, None] * g4[:, t, :, None, :] + d4[:, t, :, :, None] * A
    sh = (B, T, C)
    return gr.reshape(sh), gk.reshape(sh), gv.reshape(sh), gw.reshape(sh), gu


def make_inputs(B, T, H, N, seed=0, with_state=False, kinds=None):
    """Seeded synthetic inputs with the value distributions of the benchmark
    configurations: r,k,v ~ N(0,1)/sqrt(N); w ~ U(-6,1); u ~ N(0,0.1) [H,N];
    gy ~ N(0,1).  float32 values held in float32 arrays.
    """
    rng = np.random.default_rng(seed)
    C = H * N
    s = 1.0 / np.sqrt(N)
    out = {
        "r": (rng.standard_normal((B, T, C)) * s).astype(np.float32),
        "k": (rng.standard_normal((B, T, C)) * s).astype(np.float32),
        "v": (rng.standard_normal((B, T, C)) * s).astype(np.float32),
        "w": rng.uniform(-6.0, 1.0, (B, T, C)).astype(np.float32),
        "u": (rng.standard_normal((H, N)) * 0.1).astype(np.float32),
        "gy": rng.standard_normal((B, T, C)).astype(np.float32),
    }
    if with_state:
        kinds = B if kinds is None else kinds
        out["init_state"] = (rng.standard_normal((kinds, H, N, N)) * 0.1).astype(np.float32)
        out["state_map"] = rng.integers(0, kinds, (B,)).astype(np.int64)
    return out
