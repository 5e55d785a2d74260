"""Multi-GPU tests (skipped with fewer than two GPUs): one process per GPU over NCCL.
* B x H sharding: every rank runs its (batch, head) shard; results are bit-equal to the single-GPU run.
* T sharding: every rank holds a contiguous T range; per-head states are carried between ranks (all-gather of
  segment summaries + scan) and results match the single-GPU run within the bf16 tolerance."""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
N = 64


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, q):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        import star_rwkv6_b200 as pkg
        from star_rwkv6_b200 import segments as seg, sharding
        from oracle import wkv6_oracle as O
        B, T, H = 2, 2048, 4
        d = O.make_inputs(B, T, H, N, seed=17)
        full = {n: torch.tensor(d[n]).to(torch.bfloat16).cuda() for n in ("r", "k", "v", "w", "gy")}
        u = torch.tensor(d["u"]).cuda()
        # single-GPU reference on this rank (same kernels, unsplit)
        y1, _, ck = pkg.forward_raw(full["r"], full["k"], full["v"], full["w"], u, N, want_ckpt=True)
        g1 = pkg.backward_raw(full["r"], full["k"], full["v"], full["w"], u, full["gy"], N, ckpt=ck)
        ok = True
        # --- B x H sharding: bit-equal
        plan = sharding.make_plan(B, H, world)
        rs, ks, vs, ws, gs = (x.contiguous() for x in sharding.shard(plan, rank, N, *(full[n] for n in ("r", "k", "v", "w", "gy"))))
        us = sharding.shard_u(plan, rank, u).contiguous()
        y2, _, ck2 = pkg.forward_raw(rs, ks, vs, ws, us, N, want_ckpt=True)
        g2 = pkg.backward_raw(rs, ks, vs, ws, us, gs, N, ckpt=ck2)
        bs, cs = plan.batch_slice(rank), plan.channel_slice(rank, N)
        ok = ok and torch.equal(y2, y1[bs, :, cs])
        for a, b in zip(g2[:4], g1[:4]):
            ok = ok and torch.equal(a, b[bs, :, cs])
        gu2 = sharding.reduce_gu(plan, rank, g2[4])
        ok = ok and torch.allclose(gu2, g1[4].sum(0)[plan.head_slice(rank)], rtol=1e-5, atol=1e-6)
        # --- T sharding with carried states
        Tl = T // world
        sl = slice(rank * Tl, (rank + 1) * Tl)
        loc = {n: x[:, sl].contiguous() for n, x in full.items()}
        be = seg.LibraryBackend(N)
        y3, last, ctx = seg.segmented_forward(be, loc["r"], loc["k"], loc["v"], loc["w"], u, 2, want_ckpt=True,
                                              group=dist.group.WORLD)
        g3 = seg.segmented_backward(be, ctx, loc["r"], loc["k"], loc["v"], loc["w"], u, loc["gy"])
        torch.cuda.synchronize()

        def err(a, b):
            return float((a.float() - b.float()).abs().max() / b.float().abs().max())
        ok = ok and err(y3, y1[:, sl]) <= 1e-2
        for a, b in zip(g3[:4], g1[:4]):
            ok = ok and err(a, b[:, sl]) <= 2e-2
        ok = ok and err(g3[4], g1[4].sum(0)) <= 2e-2
        from star_rwkv6_b200 import _lib
        ok = ok and _lib.lib.wkv6_device_status() == 0
        q.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpus_sharded():
    import torch.multiprocessing as mp
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=300)
        assert p.exitcode == 0
    results = dict(q.get(timeout=10) for _ in range(world))
    assert all(results.values()), results
