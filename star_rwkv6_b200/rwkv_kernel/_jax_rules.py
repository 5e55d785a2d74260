"""Framework-free pieces of the JAX operator (no ``import jax`` here, so that they can be tested without JAX):
the shapes of the two extra buffers the chunked kernels need, the state-map dtype rule and the partitioning rule
of the op over a device mesh.

Partitioning rule (the reference imports ``custom_partitioning`` and never gives it a rule,
rwkv_kernel/jax_rwkv_kernel.py:14-19): every (batch row, head) pair is an independent recurrence
(rwkv_kernel/jax_kernel/rwkv_kernels.cu:198-199), so
* dim 0 (batch) of r, k, v, w, gy, y and of every gradient may be split over any mesh axes;
* dim 2 (channels) may be split in multiples of the head size, i.e. into whole heads; u [H, N], gu [B, H, N], the
  checkpoints [B, H, ., .] and the scratch [B, H, .] follow on their head dimension;
* dim 1 (time) is never split: a spec that shards it is replaced by a replicated time axis.
The op then runs shard-locally with no collective; gu stays per batch row and is summed by the caller.
"""
from __future__ import annotations

from typing import Optional, Sequence, Tuple

CHUNK = 64


def uses_chunked_kernels(dtype_name: str, head_size: int) -> bool:
    return dtype_name == "bfloat16" and head_size == 64


def ckpt_shape(B: int, T: int, H: int, N: int, dtype_name: str) -> Tuple[Tuple[int, ...], str]:
    """Shape and dtype of the checkpoint buffer (extra result of the forward, residual of the vjp)."""
    if uses_chunked_kernels(dtype_name, N) and T >= 1:
        return (B, H, (T + CHUNK - 1) // CHUNK, 4096), "bfloat16"
    return (B, H, 1, 8), "bfloat16"          # a placeholder the handlers ignore


def ws_shape(B: int, T: int, H: int, N: int, dtype_name: str) -> Tuple[Tuple[int, ...], str]:
    """Shape and dtype of the scratch buffer (extra result of the backward)."""
    if uses_chunked_kernels(dtype_name, N) and T >= 1:
        return (B, H, 64), "int32"           # 256 bytes per sequence: at least one flag word each, rounded up
    if dtype_name in ("float32", "float16"):
        return (B, H, 4), "int32"            # fp32 outputs: dense problems stage inside gw, a placeholder suffices
    return (B, H, max(T, 1) * N), "float32"  # the sequential variant's x_t = r_t gr_t, one value per (token, channel)


def check_state_map_dtype(dtype_name: str) -> None:
    """The handlers read ``state_map`` as int64[B].  JAX silently narrows int64 to int32 unless x64 is enabled, which
    would make the kernel read past the map; refuse instead."""
    if dtype_name != "int64":
        raise TypeError(f"state_map arrived as {dtype_name}: the kernels read int64. Enable 64-bit types "
                        "(jax.config.update('jax_enable_x64', True)) before building the map.")


def _axes(entry) -> Tuple[str, ...]:
    if entry is None:
        return ()
    return tuple(entry) if isinstance(entry, (tuple, list)) else (entry,)


def wkv_partition_specs(spec: Sequence, mesh_axis_sizes: dict, C: int, head_size: int):
    """From the PartitionSpec entries of r ([B, T, C]) to the specs the op is run with.

    Returns (x_spec, u_spec, bh_spec): entries for the [B, T, C] tensors, for u [H, N], and the leading (batch, head)
    entries of gu / ckpt / ws.  The time entry is dropped (replicated); the channel entry is kept only if it cuts C
    into whole heads."""
    spec = list(spec) + [None] * (3 - len(spec))
    b_axes, c_axes = spec[0], spec[2]
    parts = 1
    for ax in _axes(c_axes):
        parts *= int(mesh_axis_sizes[ax])
    H = C // head_size
    if parts > 1 and H % parts != 0:
        c_axes = None                         # would cut through a head: keep the channels together
    return (b_axes, None, c_axes), (c_axes, None), (b_axes, c_axes)
