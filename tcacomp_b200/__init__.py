"""tcacomp_b200 -- B200 (sm_100a) kernels for tcacomp's map / reduce / contraction path.

The product is libtcab.so (CUDA kernels behind the C ABI of include/tcab.h).
This package is the thin Python host over it: torch supplies device memory and
streams, every operator below is one C-ABI call. Nothing here computes on the
CPU and nothing falls back to torch.
"""
from . import _lib
from .ops import (BoundChainReduce, chain_contract, chain_prepare, chain_reduce, chain_reduce_batched, release_all, release_stream, chain_reduce_noalloc, device_status, gemm_bias_act, launch_count, layernorm_rows, map, reduce_outer,
                  softmax_rows, tune)
from ._lib import TcabError

__all__ = ["BoundChainReduce", "chain_contract", "chain_prepare", "chain_reduce", "chain_reduce_batched", "release_all", "release_stream", "chain_reduce_noalloc", "device_status", "gemm_bias_act", "launch_count", "layernorm_rows", "map", "reduce_outer",
           "softmax_rows", "tune", "TcabError"]
