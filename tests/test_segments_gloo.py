"""CPU tier, world_size 2 over gloo: the T-sharded path (segment summaries -> all-gather -> scan -> seeded kernels).
The numerical backend here is the float64 oracle; what is under test is the orchestration in
star_rwkv6_b200/segments.py: segment order after the gather, scan direction, slicing back, gu reduction."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import wkv6_oracle as O


class OracleBackend:
    """The segments.py backend protocol on numpy float64 (slow, tiny shapes only)."""

    def __init__(self, N):
        self.N = N

    def summary(self, x1, x2, w, reverse):
        Bn, T, C = x1.shape
        N = self.N
        H = C // N
        x1n, x2n = x1.numpy().reshape(Bn, T, H, N), x2.numpy().reshape(Bn, T, H, N)
        lw2 = (-np.exp(w.numpy().astype(np.float64)) * np.log2(np.e)).reshape(Bn, T, H, N)
        S = np.zeros((Bn, H, N, N))
        order = range(T - 1, -1, -1) if reverse else range(T)
        for t in order:
            d = np.exp2(lw2[:, t])[..., None]
            outer = x1n[:, t, :, :, None] * x2n[:, t, :, None, :]
            S = d * S + outer if not reverse else d * S + outer  # same recurrence, walked from the other end
        return torch.tensor(S), torch.tensor(lw2.sum(1))

    def scan(self, B, H, G, dec, state, s0, reverse):
        N = self.N
        dec, state = dec.numpy().reshape(B, G, H, N), state.numpy().reshape(B, G, H, N, N)
        out = np.zeros_like(state)
        S = np.zeros((B, H, N, N)) if (s0 is None or reverse) else s0.numpy().astype(np.float64)
        for g in (range(G - 1, -1, -1) if reverse else range(G)):
            out[:, g] = S
            S = np.exp2(dec[:, g])[..., None] * S + state[:, g]
        return torch.tensor(out.reshape(B * G, H, N, N)), torch.tensor(S)

    def forward(self, r, k, v, w, u, s_in, want_ckpt):
        y, _ = O.wkv6_forward(r.numpy(), k.numpy(), v.numpy(), w.numpy(), u.numpy(), self.N, init_state=s_in.numpy())
        return torch.tensor(y), s_in  # the "checkpoint" of this backend is the entering state itself

    def backward(self, r, k, v, w, u, gy, ckpt, ab_in):
        # gradients of one segment with an entering forward state (ckpt) and an entering reverse state (ab_in):
        # run the oracle's closed forms with those boundary conditions
        rn, kn, vn, wn, gn = (x.numpy().astype(np.float64) for x in (r, k, v, w, gy))
        Bn, T, C = rn.shape
        N = self.N
        H = C // N
        un = u.numpy().astype(np.float64).reshape(H, N)
        r4, k4, v4, g4 = (x.reshape(Bn, T, H, N) for x in (rn, kn, vn, gn))
        ew = np.exp(wn.reshape(Bn, T, H, N))
        d4 = np.exp(-ew)
        S = ckpt.numpy().astype(np.float64).copy()
        Sp = np.empty((T, Bn, H, N, N))
        gr = np.empty_like(r4)
        gu = np.zeros((Bn, H, N))
        for t in range(T):
            Sp[t] = S
            vg = (v4[:, t] * g4[:, t]).sum(-1)
            gr[:, t] = un[None] * k4[:, t] * vg[..., None] + np.einsum("bhij,bhj->bhi", S, g4[:, t])
            gu += r4[:, t] * k4[:, t] * vg[..., None]
            S = d4[:, t, :, :, None] * S + k4[:, t, :, :, None] * v4[:, t, :, None, :]
        A = ab_in.numpy().astype(np.float64).copy()
        gk, gv, gw = np.empty_like(r4), np.empty_like(r4), np.empty_like(r4)
        for t in range(T - 1, -1, -1):
            M = (un[None] * r4[:, t])[..., None] * g4[:, t, :, None, :] + A
            gk[:, t] = np.einsum("bhij,bhj->bhi", M, v4[:, t])
            gv[:, t] = np.einsum("bhij,bhi->bhj", M, k4[:, t])
            gw[:, t] = -ew[:, t] * d4[:, t] * np.einsum("bhij,bhij->bhi", Sp[t], A)
            A = r4[:, t, :, :, None] * g4[:, t, :, None, :] + d4[:, t, :, :, None] * A
        sh = (Bn, T, C)
        return tuple(torch.tensor(x.reshape(sh)) for x in (gr, gk, gv, gw)) + (torch.tensor(gu),)


class LeanOracleBackend(OracleBackend):
    """The same backend offering the scan-only summaries: the segment no exclusive scan reads (the last of a sequence going
    forward, the first in reverse) comes back as NaN, so any use of it poisons the results."""
    scan_only_summaries = True

    def summary(self, x1, x2, w, reverse, scan_only_segments=0):
        S, dec = super().summary(x1, x2, w, reverse)
        if scan_only_segments > 0:
            G = scan_only_segments
            rows = torch.arange(S.shape[0]) % G == (0 if reverse else G - 1)
            S[rows] = float("nan")
            dec[rows] = float("nan")
        return S, dec

    def scan(self, B, H, G, dec, state, s0, reverse):
        # like the library's kernel, the scan folds the last summary it walks over only into the state it returns second
        out, last = super().scan(B, H, G, torch.nan_to_num(dec, nan=0.0), torch.nan_to_num(state, nan=0.0), s0, reverse)
        assert not torch.isnan(out).any()
        return out, last


@pytest.mark.parametrize("G", [2, 3])
def test_lean_orchestration_single_rank(G):
    """need_last=False on one rank: no final state comes back, the skipped summaries are never needed, and the backward takes
    its decays from the reverse summaries.  The NaN rows must not reach a result... and, to make sure the scan is not fed a
    wrong row instead, the scan of this backend replaces only NaN by zero: a misplaced skip would change the numbers."""
    from star_rwkv6_b200 import segments as seg
    B, T, H, N = 2, 24, 2, 8
    d = O.make_inputs(B, T, H, N, seed=6)
    full = {n: torch.tensor(d[n], dtype=torch.float64) for n in ("r", "k", "v", "w", "gy")}
    u = torch.tensor(d["u"], dtype=torch.float64)
    be = LeanOracleBackend(N)
    y, last, ctx = seg.segmented_forward(be, full["r"], full["k"], full["v"], full["w"], u, G, want_ckpt=True, need_last=False)
    assert last is None and ctx["lean"]
    g = seg.segmented_backward(be, ctx, full["r"], full["k"], full["v"], full["w"], u, full["gy"])
    yo, _ = O.wkv6_forward(d["r"], d["k"], d["v"], d["w"], d["u"], N)
    go = O.wkv6_backward(d["r"], d["k"], d["v"], d["w"], d["u"], d["gy"], N)
    assert np.allclose(y.numpy(), yo, rtol=1e-10, atol=1e-12)
    for a, b in zip(g[:4], go[:4]):
        assert np.allclose(a.numpy(), b, rtol=1e-9, atol=1e-11)
    assert np.allclose(g[4].numpy(), go[4].sum(0), rtol=1e-9, atol=1e-11)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _run(rank, world, port, q, G):
    from star_rwkv6_b200 import segments as seg
    group = None
    if world > 1:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        dist.init_process_group("gloo", rank=rank, world_size=world)
        group = dist.group.WORLD
    try:
        B, T, H, N = 2, 24, 2, 8
        d = O.make_inputs(B, T, H, N, seed=5)
        full = {n: torch.tensor(d[n], dtype=torch.float64) for n in ("r", "k", "v", "w", "gy")}
        u = torch.tensor(d["u"], dtype=torch.float64)
        Tl = T // world
        loc = {n: x[:, rank * Tl:(rank + 1) * Tl].contiguous() for n, x in full.items()}
        be = OracleBackend(N)
        y, last, ctx = seg.segmented_forward(be, loc["r"], loc["k"], loc["v"], loc["w"], u, G, want_ckpt=True, group=group)
        g = seg.segmented_backward(be, ctx, loc["r"], loc["k"], loc["v"], loc["w"], u, loc["gy"])
        yo, so = O.wkv6_forward(d["r"], d["k"], d["v"], d["w"], d["u"], N)
        go = O.wkv6_backward(d["r"], d["k"], d["v"], d["w"], d["u"], d["gy"], N)
        sl = slice(rank * Tl, (rank + 1) * Tl)
        ok = np.allclose(y.numpy(), yo[:, sl], rtol=1e-10, atol=1e-12)
        ok = ok and np.allclose(last.numpy(), so, rtol=1e-10, atol=1e-12)
        for a, b in zip(g[:4], go[:4]):
            ok = ok and np.allclose(a.numpy(), b[:, sl], rtol=1e-9, atol=1e-11)
        ok = ok and np.allclose(g[4].numpy(), go[4].sum(0), rtol=1e-9, atol=1e-11)
        q.put((rank, bool(ok)))
    finally:
        if world > 1:
            dist.destroy_process_group()


@pytest.mark.parametrize("world,G", [(1, 3), (2, 1), (2, 2)])
def test_t_sharded_orchestration(world, G):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_run, args=(r, world, port, q, G)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=180)
        assert p.exitcode == 0
    results = dict(q.get(timeout=10) for _ in range(world))
    assert all(results[r] for r in range(world)), results
