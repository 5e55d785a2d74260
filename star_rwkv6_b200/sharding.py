"""Partitioning of the WKV6 work over the GPUs of one box.

Every (batch row, head) pair is an independent recurrence (the reference launches one CTA per pair,
rwkv_kernel/jax_kernel/rwkv_kernels.cu:198-199), so a world of G ranks splits the B*H pairs with no data-path
collective: batch rows first (contiguous slices of [B,T,C]), then heads (column ranges of the channel axis, passed
to the kernels as a row stride, no copy).  ``u`` and ``gu`` follow the head split; ``gu`` is produced per batch row
and the batch sum - an all-reduce across batch shards - belongs to the caller, as in the reference
(jax_rwkv_kernel.py:166, torch_rwkv_kernel.py:73).  This is the rule a ``custom_partitioning`` /
``shard_map`` wrapper applies (see rwkv_kernel/jax_rwkv_kernel.py).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Tuple


@dataclass(frozen=True)
class Plan:
    B: int
    H: int
    world: int
    batch_parts: int   # ranks along the batch axis
    head_parts: int    # ranks along the head axis

    def coords(self, rank: int) -> Tuple[int, int]:
        assert 0 <= rank < self.world
        return rank // self.head_parts, rank % self.head_parts

    def batch_slice(self, rank: int) -> slice:
        bi, _ = self.coords(rank)
        per = self.B // self.batch_parts
        return slice(bi * per, (bi + 1) * per)

    def head_slice(self, rank: int) -> slice:
        _, hi = self.coords(rank)
        per = self.H // self.head_parts
        return slice(hi * per, (hi + 1) * per)

    def channel_slice(self, rank: int, head_size: int) -> slice:
        hs = self.head_slice(rank)
        return slice(hs.start * head_size, hs.stop * head_size)

    def local_shape(self) -> Tuple[int, int]:
        return self.B // self.batch_parts, self.H // self.head_parts


def make_plan(B: int, H: int, world: int) -> Plan:
    """Split B*H pairs over ``world`` ranks: as many ranks as divide B go to the batch axis, the rest to heads."""
    if world < 1:
        raise ValueError("world must be >= 1")
    bp = 1
    for cand in range(min(B, world), 0, -1):
        if B % cand == 0 and world % cand == 0:
            bp = cand
            break
    hp = world // bp
    if H % hp != 0:
        raise ValueError(f"cannot split B={B}, H={H} evenly over {world} ranks")
    return Plan(B, H, world, bp, hp)


def shard(plan: Plan, rank: int, head_size: int, *tensors):
    """Views of [B,T,C] tensors for ``rank`` (no copy; a head split yields a strided view)."""
    bs, cs = plan.batch_slice(rank), plan.channel_slice(rank, head_size)
    return tuple(t[bs, :, cs] for t in tensors)


def shard_u(plan: Plan, rank: int, u):
    return u[plan.head_slice(rank)]


def reduce_gu(plan: Plan, rank: int, gu_rows, group=None):
    """Batch-sum of the per-row ``gu`` [B_local, H_local, N] -> [H_local, N] for this rank's heads: a local sum
    followed by an all-reduce over the ranks that hold the other batch rows of the same heads."""
    import torch
    import torch.distributed as dist
    g = gu_rows.sum(0)
    if plan.batch_parts > 1:
        if plan.head_parts == 1:
            dist.all_reduce(g, op=dist.ReduceOp.SUM, group=group)
        else:
            # ranks with the same head coordinate form one reduction group; gather-and-mask keeps this helper
            # free of sub-group bookkeeping
            _, hi = plan.coords(rank)
            parts = [torch.zeros_like(g) for _ in range(plan.world)]
            dist.all_gather(parts, g.contiguous(), group=group)
            g = sum(p for r2, p in enumerate(parts) if plan.coords(r2)[1] == hi)
    return g
