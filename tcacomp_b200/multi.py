"""One benchmark-sized problem partitioned over N GPUs along its independent axis.

Two forms, both without a data-path collective:
  * several devices in ONE process: `pipeline.MultiDevice` (the library's tcab_multi driver);
  * one process per GPU (torchrun): rank r of W takes `shard.block(units, W, r)` of the same global problem
    and runs it through its own `pipeline.Pipeline` -- `run_block` below. Replicated operands (gamma / beta,
    b / bias) are copied into each GPU's memory by the caller before timing.
The reference has nothing comparable: it spreads loop dims over the CTAs and warps of one GPU
(internal/cg/cxx/loops.go:11-22).
"""
from __future__ import annotations

from typing import Sequence, Tuple

import torch

from .pipeline import Pipeline
from .shard import block


def block_views(tensors: Sequence[torch.Tensor], units: int, world: int, rank: int) -> Tuple[list, int]:
    """This rank's block of every tensor whose leading extent is the independent axis, and its length."""
    lo, hi = block(units, world, rank)
    return [t[lo:hi] for t in tensors], hi - lo


def run_block(pipe: Pipeline, host_ins: Sequence[torch.Tensor], host_outs: Sequence[torch.Tensor], units: int,
              world: int, rank: int) -> int:
    """Queue rank `rank`'s block of a global problem of `units` units held in host memory; returns its length.

    host_ins / host_outs are the GLOBAL buffers (leading extent = units); only the block's slices are read and
    written, so every rank may pass the same shared buffers or its own."""
    ins, n = block_views(host_ins, units, world, rank)
    outs, _ = block_views(host_outs, units, world, rank)
    if n > 0:
        pipe.run(ins, outs, n)
    return n
