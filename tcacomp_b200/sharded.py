"""Reductions ALONG a sharded axis: the one place where the path needs a collective.

When t[b, k, c] is sharded over k (each rank holds a contiguous block of k), the outer-axis reduce
becomes: local partial (sum, max, argmax) on each GPU with the ordinary kernel, then an exchange:
  * sum: all-reduce(SUM) of the partial sums;
  * max: all-reduce(MAX) of the partial maxima;
  * argmax: the partial argmax is made global (local index + the rank's k offset); among the ranks
    whose partial max equals the global max the LOWEST global index wins, which is an
    all-reduce(MIN) over "index if my max is the global max, else a sentinel".
Three small collectives on [b, c] tensors (NCCL over NVLink on GPUs, gloo on CPU for the tests); the
[b, k, c] data itself never moves. The reference has nothing comparable: its multi-CTA reducer is a
stub (runtime/tca/reducer.h:187-213) and it has no multi-device support at all.

The tie rule matches the single-GPU kernel and the oracle: lowest index among equal maxima; a NaN
never wins, and a column that is NaN or -inf everywhere keeps index 0.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch
import torch.distributed as dist

_SENTINEL = 2**31 - 1


def combine_partials(partial: Dict[str, torch.Tensor], k_offset: int,
                     group: Optional[dist.ProcessGroup] = None) -> Dict[str, torch.Tensor]:
    """Combine per-rank partial results of a k-sharded outer reduce in place and return them.

    partial: any of {"sum", "max", "argmax"} as produced by reduce_outer on the local k block;
    "argmax" requires "max". k_offset: the global index of this rank's first k.
    """
    if "sum" in partial:
        dist.all_reduce(partial["sum"], op=dist.ReduceOp.SUM, group=group)
    if "argmax" in partial and "max" not in partial:
        raise ValueError("combining a sharded argmax needs the partial max as well")
    if "max" in partial:
        local_max = partial["max"].clone() if "argmax" in partial else None
        dist.all_reduce(partial["max"], op=dist.ReduceOp.MAX, group=group)
        if "argmax" in partial:
            gmax = partial["max"]
            # -inf everywhere (or NaN everywhere: the partial max is then -inf too) keeps index 0
            mine = (local_max == gmax) & (gmax > float("-inf"))
            cand = torch.where(mine, partial["argmax"] + k_offset, torch.full_like(partial["argmax"], _SENTINEL))
            dist.all_reduce(cand, op=dist.ReduceOp.MIN, group=group)
            partial["argmax"].copy_(torch.where(cand == _SENTINEL, torch.zeros_like(cand), cand))
    return partial


def reduce_outer_sharded_k(t_local: torch.Tensor, k_offset: int, want=("sum", "max", "argmax"),
                           group: Optional[dist.ProcessGroup] = None) -> Dict[str, torch.Tensor]:
    """sum / max / argmax over the GLOBAL k of a tensor whose k axis is sharded across the group.

    t_local: this rank's [b, k_local, c] block (CUDA, fp32). Every rank returns the full result.
    """
    from .ops import reduce_outer
    need = set(want) | ({"max"} if "argmax" in want else set())
    part = reduce_outer(t_local, want=tuple(sorted(need)))
    out = combine_partials(part, k_offset, group)
    return {k: out[k] for k in want}
