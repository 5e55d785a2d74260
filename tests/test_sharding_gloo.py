"""CPU tier, world_size 2 over gloo: the partition rule of the multi-GPU path.  The compute of each rank is the
oracle here (no GPU in this tier); what is checked is that shard-local results reassemble to the unsharded ones,
that gu is reduced over batch shards only, and the bench's max-over-ranks timing reduction."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import wkv6_oracle as O
from star_rwkv6_b200 import sharding


def test_plans():
    p = sharding.make_plan(8, 32, 8)
    assert (p.batch_parts, p.head_parts) == (8, 1) and p.local_shape() == (1, 32)
    p = sharding.make_plan(2, 32, 8)
    assert (p.batch_parts, p.head_parts) == (2, 4) and p.local_shape() == (1, 8)
    p = sharding.make_plan(1, 32, 4)
    assert (p.batch_parts, p.head_parts) == (1, 4)
    covered = set()
    p = sharding.make_plan(4, 6, 6)
    for r in range(6):
        bs, hs = p.batch_slice(r), p.head_slice(r)
        for b in range(bs.start, bs.stop):
            for h in range(hs.start, hs.stop):
                assert (b, h) not in covered
                covered.add((b, h))
    assert len(covered) == 24
    with pytest.raises(ValueError):
        sharding.make_plan(3, 5, 4)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, B, H, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        N, T = 8, 12
        d = O.make_inputs(B, T, H, N, seed=71)
        plan = sharding.make_plan(B, H, world)
        full = {n: torch.tensor(d[n]) for n in ("r", "k", "v", "w", "gy")}
        r, k, v, w, gy = sharding.shard(plan, rank, N, *(full[n] for n in ("r", "k", "v", "w", "gy")))
        u = sharding.shard_u(plan, rank, torch.tensor(d["u"]))
        y, _ = O.wkv6_forward(r.numpy(), k.numpy(), v.numpy(), w.numpy(), u.numpy(), N)
        g = O.wkv6_backward(r.numpy(), k.numpy(), v.numpy(), w.numpy(), u.numpy(), gy.numpy(), N)
        gu = sharding.reduce_gu(plan, rank, torch.tensor(g[4]))
        # reassemble on every rank
        Bl, Hl = plan.local_shape()
        outs = {}
        for name, loc in (("y", y), ("gr", g[0]), ("gk", g[1]), ("gv", g[2]), ("gw", g[3])):
            parts = [torch.zeros((Bl, T, Hl * N), dtype=torch.float64) for _ in range(world)]
            dist.all_gather(parts, torch.tensor(loc).contiguous())
            whole = torch.zeros((B, T, H * N), dtype=torch.float64)
            for r2, p in enumerate(parts):
                whole[plan.batch_slice(r2), :, plan.channel_slice(r2, N)] = p
            outs[name] = whole.numpy()
        gparts = [torch.zeros_like(gu) for _ in range(world)]
        dist.all_gather(gparts, gu.contiguous())
        gu_full = torch.zeros((H, N), dtype=torch.float64)
        for r2, p in enumerate(gparts):
            gu_full[plan.head_slice(r2)] = p
        # the timing reduction used by bench.py: max over ranks
        tt = torch.tensor([1.0 + rank], dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        if rank == 0:
            yo, _ = O.wkv6_forward(d["r"], d["k"], d["v"], d["w"], d["u"], N)
            go = O.wkv6_backward(d["r"], d["k"], d["v"], d["w"], d["u"], d["gy"], N)
            ok = np.allclose(outs["y"], yo, rtol=1e-12, atol=1e-14)
            for name, ref in zip(("gr", "gk", "gv", "gw"), go[:4]):
                ok = ok and np.allclose(outs[name], ref, rtol=1e-12, atol=1e-14)
            ok = ok and np.allclose(gu_full.numpy(), go[4].sum(0), rtol=1e-12, atol=1e-14)
            ok = ok and tt.item() == float(world)
            q.put(bool(ok))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("B,H", [(2, 2), (1, 4), (3, 2)])
def test_two_ranks_reassemble(B, H):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, B, H, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert q.get(timeout=10) is True
