"""How the GEMM is divided across the GPUs of one box (one process per GPU).

Row sharding: rank g owns a contiguous block of rows of A and C, B is replicated; the ranks
never exchange data.  Split-K: rank g owns one or more consecutive K slices of A and B, computes
a full-size int32 partial and the partials are summed by one reduce-scatter, after which rank g
holds row block g of C.
"""
from __future__ import annotations


def row_shard(m: int, world: int, rank: int) -> tuple[int, int]:
    """(first_row, n_rows) of rank `rank`; blocks differ by at most one row and cover [0, m)."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError("row_shard: bad world/rank")
    base, extra = divmod(m, world)
    rows = base + (1 if rank < extra else 0)
    first = rank * base + min(rank, extra)
    return first, rows


def k_slices(splitk: int, world: int, rank: int) -> range:
    """Indices of the K slices rank `rank` accumulates locally (splitk must be a multiple of world)."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError("k_slices: bad world/rank")
    if splitk % world:
        raise ValueError("k_slices: splitk must be a multiple of the number of ranks")
    per = splitk // world
    return range(rank * per, (rank + 1) * per)


def k_range(k: int, splitk: int, world: int, rank: int) -> tuple[int, int]:
    """(first_k, n_k) covered by the slices of `rank` (equal contiguous slices, splitk divides k)."""
    if k % splitk:
        raise ValueError("k_range: splitk must divide K")
    sl = k_slices(splitk, world, rank)
    ks = k // splitk
    return sl.start * ks, len(sl) * ks
