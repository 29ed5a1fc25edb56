"""Sharding of the attention path across ranks (one process per GPU).

The ranks form batch_groups x head_groups (rank = batch_index * head_groups +
head_index).  A batch group owns batch / batch_groups of the batch items (the
branches of classifier-free guidance are independent forwards); inside it rank g
of G owns head columns [g*H/G, (g+1)*H/G) of q, k, v.  Nothing is exchanged before
attention; afterwards only the head columns travel, inside a batch group.

NCCL comparison path (one batch group):  Per layer the ranks' outputs
[rows, (H/G)*128] are gathered: the collective lands them rank-major,
[G][rows][slice], and an interleave pass produces the token-major
[rows, H*128] tensor the next op of the block expects.
"""
from __future__ import annotations

import numpy as np


def head_range(rank: int, world: int, heads: int) -> tuple[int, int]:
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world {world}")
    if heads % world:
        raise ValueError(f"{heads} heads do not shard over {world} ranks")
    per = heads // world
    return rank * per, (rank + 1) * per


def shard_heads(x: np.ndarray, rank: int, world: int) -> np.ndarray:
    """x: [..., heads, 128] -> this rank's contiguous head slice."""
    lo, hi = head_range(rank, world, x.shape[-2])
    return np.ascontiguousarray(x[..., lo:hi, :])


def interleave(staged: np.ndarray, rows: int, slice_elements: int, world: int) -> np.ndarray:
    """Rank-major landing zone [world][rows][slice] -> token-major [rows][world*slice]
    (what qw_gpu_group_all_gather_heads_bf16 leaves in `full`)."""
    staged = np.asarray(staged).reshape(world, rows, slice_elements)
    return np.ascontiguousarray(staged.transpose(1, 0, 2)).reshape(rows, world * slice_elements)


def layout(rank: int, world: int, batch: int, batch_groups: int = 1):
    """(batch_index, head_index, head_groups, first batch item, batch items) of a rank."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world {world}")
    if batch_groups < 1 or world % batch_groups or batch % batch_groups:
        raise ValueError(f"{world} ranks / batch {batch} do not split into {batch_groups} batch groups")
    head_groups = world // batch_groups
    per = batch // batch_groups
    batch_index, head_index = divmod(rank, head_groups)
    return batch_index, head_index, head_groups, batch_index * per, per


def default_batch_groups(world: int, batch: int) -> int:
    """Split by batch item first (no exchange at all between the guidance
    branches), then by head: the largest divisor of both."""
    groups = 1
    for g in range(1, batch + 1):
        if batch % g == 0 and world % g == 0:
            groups = g
    return groups


def shard(x: np.ndarray, rank: int, world: int, batch_groups: int = 1) -> np.ndarray:
    """x: [batch, rows, heads, 128] -> this rank's [batch items, rows, local heads, 128]."""
    _, head_index, head_groups, b0, nb = layout(rank, world, x.shape[0], batch_groups)
    lo, hi = head_range(head_index, head_groups, x.shape[-2])
    return np.ascontiguousarray(x[b0:b0 + nb, :, lo:hi, :])
