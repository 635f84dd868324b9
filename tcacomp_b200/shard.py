"""Partitioning of the independent axis (rows / batch / M) across ranks.

Every operator class here has an axis along which outputs are independent, so
multi-GPU execution is a pure partition: rank r of W owns one contiguous block
of that axis and no data-path collective is needed. (The reference has no
multi-device support at all; it only spreads loop dims over CTAs and warps,
internal/cg/cxx/loops.go:11-22.)
"""
from __future__ import annotations

from typing import List, Tuple


def block(n: int, world: int, rank: int) -> Tuple[int, int]:
    """[lo, hi) of the contiguous block rank `rank` owns out of n units.

    Blocks differ in size by at most one unit; the first n % world ranks get
    the larger ones. Every unit belongs to exactly one rank.
    """
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} of {world}")
    if n < 0:
        raise ValueError("negative extent")
    base, extra = divmod(n, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def blocks(n: int, world: int) -> List[Tuple[int, int]]:
    return [block(n, world, r) for r in range(world)]
