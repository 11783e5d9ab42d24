"""Sharding of the operator across GPUs: the (batch, head) pairs of one call are independent, so
rank r of W takes a contiguous slice of the flattened pair index and no collective is involved."""
from __future__ import annotations


def shard_pairs(B: int, H: int, rank: int, world: int) -> tuple[int, int]:
    """[lo, hi) slice of the B*H flattened (batch, head) pairs owned by `rank`; sizes differ by at most one."""
    n = B * H
    base, extra = divmod(n, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def shard_batch_rows(B: int, rank: int, world: int) -> tuple[int, int]:
    """[lo, hi) slice of batch rows for weak-/strong-scaling runs that shard whole sequences."""
    base, extra = divmod(B, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)
