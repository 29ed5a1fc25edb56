"""Head sharding of the attention path across ranks (one process per GPU).

Rank g of G owns head columns [g*H/G, (g+1)*H/G) of q, k, v for every batch item;
nothing is exchanged before attention.  Per layer the ranks' outputs
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
