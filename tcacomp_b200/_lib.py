"""ctypes view of libtcab.so, one-to-one with include/tcab.h.

The library is never substituted: if libtcab.so is missing or does not load,
importing this module raises, and so does every operator.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libtcab.so")

MAX_RANK = 4
MAX_INPUTS = 6
MAX_CAPTURES = 8
NOALLOC_MAX_ROWS = 4096
MAX_BATCH = 32

OK, ERR_INVALID_ARG, ERR_SHAPE, ERR_DTYPE, ERR_ALIGNMENT, ERR_UNSUPPORTED, ERR_CUDA, ERR_TOO_LARGE = range(8)
F32, BF16, I32, U32 = 0, 1, 2, 3
ACT_NONE, ACT_RELU = 0, 1
USE_REDUCE, USE_CONTRACT, USE_MAP, USE_REDUCE_BATCHED = 0, 1, 2, 3


class Tensor(C.Structure):
    """tcab_tensor: a non-owning view (device pointer, dtype, rank, extents)."""
    _fields_ = [("data", C.c_void_p), ("dtype", C.c_int32), ("rank", C.c_uint32),
                ("dims", C.c_uint32 * MAX_RANK)]


class Chain(C.Structure):
    """tcab_chain: map | reduce | map lambdas as canonical C expressions."""
    _fields_ = [("map_expr", C.c_char_p), ("combine_expr", C.c_char_p), ("post_expr", C.c_char_p),
                ("init", C.c_float), ("n_captures", C.c_uint32), ("captures", C.c_float * MAX_CAPTURES)]


class PipelineDesc(C.Structure):
    """tcab_pipeline_desc: one operator over host buffers, cut into chunks of its independent axis."""
    _fields_ = [("op", C.c_int32), ("device", C.c_int32), ("chunk_units", C.c_uint32), ("depth", C.c_uint32),
                ("in_dtype", C.c_int32), ("n_streamed", C.c_uint32), ("unit_rank", C.c_uint32),
                ("unit_dims", C.c_uint32 * (MAX_RANK - 1)), ("outputs", C.c_uint32), ("out_dtype", C.c_int32),
                ("act", C.c_int32), ("eps", C.c_float), ("chain", C.POINTER(Chain)), ("resident", Tensor * 2)]


OP_SOFTMAX_ROWS, OP_LAYERNORM_ROWS, OP_REDUCE_OUTER, OP_CHAIN_REDUCE, OP_GEMM_BIAS_ACT, OP_MAP = range(6)


class TcabError(RuntimeError):
    """A non-zero status from the C ABI; carries the status and the library's message."""

    def __init__(self, status: int, message: str):
        super().__init__(f"tcab status {status}: {message}")
        self.status = status
        self.message = message


# Every symbol include/tcab.h declares: (name, restype, argtypes).
SYMBOLS = [
    ("tcab_last_error", C.c_char_p, []),
    ("tcab_status_string", C.c_char_p, [C.c_int]),
    ("tcab_abi_version", C.c_int, []),
    ("tcab_launch_count", C.c_uint64, []),
    ("tcab_chain_reduce", C.c_int,
     [C.POINTER(Chain), C.POINTER(Tensor), C.c_uint32, C.c_uint32, C.POINTER(Tensor), C.c_void_p]),
    ("tcab_chain_reduce_batched", C.c_int,
     [C.POINTER(Chain), C.POINTER(Tensor), C.c_uint32, C.c_uint32, C.POINTER(Tensor), C.c_void_p]),
    ("tcab_chain_reduce_noalloc", C.c_int,
     [C.POINTER(Chain), C.POINTER(Tensor), C.c_uint32, C.POINTER(Tensor), C.c_void_p]),
    ("tcab_chain_contract", C.c_int,
     [C.POINTER(Chain), C.POINTER(Tensor), C.POINTER(Tensor), C.c_int, C.POINTER(Tensor), C.c_void_p]),
    ("tcab_reduce_outer", C.c_int,
     [C.POINTER(Tensor), C.POINTER(Tensor), C.POINTER(Tensor), C.POINTER(Tensor), C.c_void_p]),
    ("tcab_softmax_rows", C.c_int, [C.POINTER(Tensor), C.POINTER(Tensor), C.c_void_p]),
    ("tcab_layernorm_rows", C.c_int,
     [C.POINTER(Tensor), C.POINTER(Tensor), C.POINTER(Tensor), C.c_float, C.POINTER(Tensor), C.c_void_p]),
    ("tcab_gemm_bias_act", C.c_int,
     [C.POINTER(Tensor), C.POINTER(Tensor), C.POINTER(Tensor), C.c_int, C.POINTER(Tensor), C.c_void_p]),
    ("tcab_device_status", C.c_int, [C.POINTER(C.c_int)]),
    ("tcab_chain_prepare", C.c_int, [C.POINTER(Chain), C.POINTER(C.c_int32), C.c_uint32, C.c_int, C.c_int]),
    ("tcab_map", C.c_int, [C.POINTER(Chain), C.POINTER(Tensor), C.c_uint32, C.POINTER(Tensor), C.c_void_p]),
    ("tcab_pipeline_create", C.c_int, [C.POINTER(PipelineDesc), C.POINTER(C.c_void_p)]),
    ("tcab_pipeline_outputs", C.c_uint32, [C.c_void_p]),
    ("tcab_pipeline_run", C.c_int, [C.c_void_p, C.POINTER(C.c_void_p), C.c_uint64, C.POINTER(C.c_void_p)]),
    ("tcab_pipeline_order_after", C.c_int, [C.c_void_p, C.c_void_p]),
    ("tcab_pipeline_join", C.c_int, [C.c_void_p, C.c_void_p]),
    ("tcab_pipeline_sync", C.c_int, [C.c_void_p]),
    ("tcab_pipeline_destroy", C.c_int, [C.c_void_p]),
    ("tcab_multi_create", C.c_int, [C.POINTER(PipelineDesc), C.c_uint32, C.POINTER(C.c_void_p)]),
    ("tcab_multi_run", C.c_int, [C.c_void_p, C.POINTER(C.c_void_p), C.c_uint64, C.POINTER(C.c_void_p)]),
    ("tcab_multi_sync", C.c_int, [C.c_void_p]),
    ("tcab_multi_destroy", C.c_int, [C.c_void_p]),
    ("tcab_shard_block", C.c_int, [C.c_uint64, C.c_uint32, C.c_uint32, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]),
    ("tcab_host_alloc", C.c_int, [C.c_uint64, C.POINTER(C.c_void_p)]),
    ("tcab_host_free", C.c_int, [C.c_void_p]),
    ("tcab_release_stream", C.c_int, [C.c_void_p]),
    ("tcab_release_all", C.c_int, []),
]

# include/tcab_tuning.h: benchmarking and test hooks, not part of the surface a host binds.
TUNING_SYMBOLS = [
    ("tcab_tune", C.c_int, [C.c_char_p, C.c_int, C.c_int, C.c_int, C.c_int]),
    ("tcab_compile_check", C.c_int,
     [C.POINTER(Chain), C.POINTER(C.c_int32), C.c_uint32, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int]),
    ("tcab_plan_row_kernels", C.c_int,
     [C.c_uint64, C.c_uint32, C.c_uint32, C.c_int, C.c_uint32, C.c_uint32, C.c_int, C.c_int, C.POINTER(C.c_uint32),
      C.POINTER(C.c_uint32), C.POINTER(C.c_uint32)]),
    ("tcab_plan_row_shape", C.c_int, [C.c_int, C.c_int, C.c_uint32, C.POINTER(C.c_uint32), C.POINTER(C.c_uint32)]),
    ("tcab_plan_outer_flat_ranges", C.c_int,
     [C.c_uint64, C.c_uint32, C.c_uint32, C.c_int, C.c_uint64, C.POINTER(C.c_uint32), C.POINTER(C.c_uint32),
      C.POINTER(C.c_uint32)]),
    ("tcab_plan_outer_split", C.c_int,
     [C.c_uint64, C.c_uint64, C.c_uint32, C.c_uint64, C.c_int, C.c_int, C.POINTER(C.c_uint32), C.POINTER(C.c_uint32)]),
]

_lib = None


def load() -> C.CDLL:
    """Load libtcab.so and bind every declared symbol; raises if anything is missing."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m tcacomp_b200.build` "
            "(there is no fallback implementation)")
    lib = C.CDLL(LIB_PATH)
    for name, restype, argtypes in SYMBOLS + TUNING_SYMBOLS:
        fn = getattr(lib, name)  # AttributeError if the library does not export it
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


def check(status: int) -> None:
    if status != OK:
        raise TcabError(status, load().tcab_last_error().decode("utf-8", "replace"))
