"""ctypes binding of oracle/liboracle.so (and oracle/_ref/libtcaref.so).

Test infrastructure only. Importers: tests/, the smoke check and the CPU
baseline leg of the benchmark. All arrays are C-contiguous numpy arrays;
bf16 data travels as uint16 bit patterns.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

from . import build as _build

_HERE = os.path.dirname(os.path.abspath(__file__))

SUITE = {
    # name: (kernel id, reduce class, dims (as the runner declares them), scalars)
    "dup_expr": (0, "inner", (256, 256, 8), (1.5, 0.25)),
    "dup_const": (1, "inner", (256, 256, 8), ()),
    "axpy3": (2, "inner", (512, 512, 4), (2.0, 0.5, 0.75)),
    "mlp": (3, "mm", (64, 128, 64), ()),
    "softmax": (4, "middle", (128, 8, 256), ()),
    "mm_small": (5, "mm", (32, 32, 32), ()),
    "mm_mid": (5, "mm", (128, 256, 64), ()),
    "mm_splitk": (5, "mm", (64, 128, 64), ()),
    "gemm": (5, "mm", (128, 128, 96), ()),
    "transpose": (6, "inner", (192, 96, 8), ()),
    "row_sum": (7, "middle", (512, 4, 1024), ()),
    "scale_copy": (8, "inner", (512, 512, 4), (1.25, -0.125)),
    "qk_score": (9, "qk", (128, 64, 192), (0.125,)),
    "layernorm": (10, "inner", (128, 256, 64), (1.0 / 64.0, 1e-5)),
}

_lib = None
_ref = None


def _ptr(a: np.ndarray | None):
    if a is None:
        return None
    assert a.flags["C_CONTIGUOUS"], "oracle arrays must be C-contiguous"
    return a.ctypes.data_as(C.c_void_p)


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        _lib = C.CDLL(_build.build_oracle())
        _lib.orc_num_threads.restype = C.c_int
        _lib.orc_suite.restype = C.c_int
    return _lib


def ref() -> C.CDLL | None:
    """The reference's runtime primitives compiled for the host, or None."""
    global _ref
    if _ref is None:
        d = _build.build_ref()
        if d is None:
            return None
        _ref = C.CDLL(os.path.join(d, "libtcaref.so"))
        _ref.ref_fold.restype = C.c_float
    return _ref


def num_threads() -> int:
    return int(lib().orc_num_threads())


def set_num_threads(n: int) -> None:
    lib().orc_set_num_threads(C.c_int(n))


def elem_fill(n: int) -> np.ndarray:
    out = np.empty(n, np.float32)
    lib().orc_elem_fill(_ptr(out), C.c_uint32(n))
    return out


def f32_to_bf16(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, np.float32)
    out = np.empty(x.shape, np.uint16)
    lib().orc_f32_to_bf16(_ptr(x), _ptr(out), C.c_uint64(x.size))
    return out


def bf16_to_f32(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, np.uint16)
    out = np.empty(x.shape, np.float32)
    lib().orc_bf16_to_f32(_ptr(x), _ptr(out), C.c_uint64(x.size))
    return out


def map_rowsum_affine_sq(x: np.ndarray, a: float = 0.5, b: float = 0.25) -> np.ndarray:
    rows, cols = x.shape
    y = np.empty(rows, np.float32)
    lib().orc_map_rowsum_affine_sq(_ptr(x), C.c_uint32(rows), C.c_uint32(cols), C.c_float(a),
                                   C.c_float(b), _ptr(y))
    return y


def map_rowsum_affine_sq_f64(x: np.ndarray, a: float = 0.5, b: float = 0.25) -> np.ndarray:
    rows, cols = x.shape
    y = np.empty(rows, np.float64)
    lib().orc_map_rowsum_affine_sq_f64(_ptr(x), C.c_uint32(rows), C.c_uint32(cols), C.c_float(a),
                                       C.c_float(b), _ptr(y))
    return y


def row_reduce(x: np.ndarray, op: str, init: float) -> np.ndarray:
    rows, cols = x.shape
    y = np.empty(rows, np.float32)
    lib().orc_row_reduce(_ptr(x), C.c_uint32(rows), C.c_uint32(cols),
                         C.c_int({"sum": 0, "max": 1, "min": 2}[op]), C.c_float(init), _ptr(y))
    return y


def softmax_rows(x: np.ndarray) -> np.ndarray:
    rows, cols = x.shape
    y = np.empty_like(x)
    lib().orc_softmax_rows(_ptr(x), C.c_uint32(rows), C.c_uint32(cols), _ptr(y))
    return y


def layernorm_rows_bf16(x: np.ndarray, gamma: np.ndarray, beta: np.ndarray,
                        eps: float = 1e-5) -> np.ndarray:
    rows, cols = x.shape
    assert x.dtype == np.uint16 and gamma.dtype == np.uint16 and beta.dtype == np.uint16
    y = np.empty_like(x)
    lib().orc_layernorm_rows_bf16(_ptr(x), _ptr(gamma), _ptr(beta), C.c_uint32(rows),
                                  C.c_uint32(cols), C.c_float(eps), _ptr(y))
    return y


def check_layernorm_bf16(got: np.ndarray, want: np.ndarray, x: np.ndarray, gamma: np.ndarray, beta: np.ndarray,
                         eps: float = 1e-5) -> np.ndarray:
    """Per-row counts [rows, 5] of the bf16 layer-norm criterion (oracle/checks.py states it):
    checked, failed, accepted only through the added terms, got != want, want != rounded fp64."""
    rows, cols = x.shape
    for a in (got, want, x, gamma, beta):
        assert a.dtype == np.uint16
    counts = np.zeros((rows, 5), np.uint64)
    lib().orc_check_layernorm_bf16(_ptr(got), _ptr(want), _ptr(x), _ptr(gamma), _ptr(beta), C.c_uint32(rows),
                                   C.c_uint32(cols), C.c_double(eps), _ptr(counts))
    return counts


def check_softmax(got: np.ndarray, want: np.ndarray, x: np.ndarray) -> np.ndarray:
    """Per-row counts [rows, 5] of the two-sided softmax criterion: checked, failed, accepted only through
    the oracle's own distance to the fp64 value (the last two columns are unused)."""
    rows, cols = x.shape
    for a in (got, want, x):
        assert a.dtype == np.float32
    counts = np.zeros((rows, 5), np.uint64)
    lib().orc_check_softmax(_ptr(got), _ptr(want), _ptr(x), C.c_uint32(rows), C.c_uint32(cols), _ptr(counts))
    return counts


def layernorm_rows_f32(x: np.ndarray, gamma: np.ndarray, beta: np.ndarray,
                       eps: float = 1e-5) -> np.ndarray:
    rows, cols = x.shape
    y = np.empty_like(x)
    lib().orc_layernorm_rows_f32(_ptr(x), _ptr(gamma), _ptr(beta), C.c_uint32(rows),
                                 C.c_uint32(cols), C.c_float(eps), _ptr(y))
    return y


def reduce_outer(t: np.ndarray):
    """(sum f32, max f32, argmax i32) of t[b, k, c] over k."""
    nb, nk, nc = t.shape
    s = np.empty((nb, nc), np.float32)
    m = np.empty((nb, nc), np.float32)
    a = np.empty((nb, nc), np.int32)
    lib().orc_reduce_outer(_ptr(t), C.c_uint32(nb), C.c_uint32(nk), C.c_uint32(nc), _ptr(s),
                           _ptr(m), _ptr(a))
    return s, m, a


def reduce_outer_sum_f64(t: np.ndarray):
    nb, nk, nc = t.shape
    s = np.empty((nb, nc), np.float64)
    sa = np.empty((nb, nc), np.float64)
    lib().orc_reduce_outer_sum_f64(_ptr(t), C.c_uint32(nb), C.c_uint32(nk), C.c_uint32(nc),
                                   _ptr(s), _ptr(sa))
    return s, sa


def gemm_bias_act_bf16(a: np.ndarray, b: np.ndarray, bias: np.ndarray | None,
                       act: str = "relu") -> np.ndarray:
    m, k = a.shape
    k2, n = b.shape
    assert k == k2 and a.dtype == np.uint16 and b.dtype == np.uint16
    c = np.empty((m, n), np.uint16)
    lib().orc_gemm_bias_act_bf16(_ptr(a), _ptr(b), _ptr(bias), C.c_uint32(m), C.c_uint32(n),
                                 C.c_uint32(k), C.c_int({"none": 0, "relu": 1}[act]), _ptr(c))
    return c


def matmul_scale_f32(lhs: np.ndarray, rhs: np.ndarray, scale: float = 1.0) -> np.ndarray:
    m, n = lhs.shape
    n2, q = rhs.shape
    assert n == n2
    out = np.empty((m, q), np.float32)
    lib().orc_matmul_scale_f32(_ptr(lhs), _ptr(rhs), C.c_uint32(m), C.c_uint32(n), C.c_uint32(q),
                               C.c_float(scale), _ptr(out))
    return out


def suite_inputs(name: str):
    """The two input tensors of a suite kernel, filled with the reference's elem(i)."""
    _, cls, (d0, d1, d2), _ = SUITE[name]
    if cls in ("inner", "middle"):
        x = elem_fill(d0 * d1 * d2).reshape(d0, d1, d2)
        return x, x.copy()
    if cls == "mm":
        return elem_fill(d0 * d1).reshape(d0, d1), elem_fill(d1 * d2).reshape(d1, d2)
    return elem_fill(d0 * d1).reshape(d0, d1), elem_fill(d2 * d1).reshape(d2, d1)  # qk


def suite(name: str, x: np.ndarray | None = None, z: np.ndarray | None = None) -> np.ndarray:
    kid, cls, (d0, d1, d2), scalars = SUITE[name]
    if x is None:
        x, z = suite_inputs(name)
    shape = (d0, d1) if cls == "inner" else (d0, d2)
    out = np.empty(shape, np.float32)
    s = np.asarray(scalars if scalars else (0.0,), np.float32)
    rc = lib().orc_suite(C.c_int(kid), _ptr(x), _ptr(z), C.c_uint32(d0), C.c_uint32(d1),
                         C.c_uint32(d2), _ptr(s), _ptr(out))
    assert rc == 0
    return out


# --- the reference's primitives on the host (None-safe callers check ref()) ---

def ref_row_sum_one_tier(lhs: np.ndarray, ctas: int = 100, threads: int = 32,
                         tile_cols: int = 64) -> np.ndarray:
    d0, d1 = lhs.shape
    out = np.full(d0, -12345.0, np.float32)
    ref().ref_row_sum_one_tier(_ptr(lhs), C.c_uint32(d0), C.c_uint32(d1), C.c_uint32(ctas),
                               C.c_uint32(threads), C.c_uint32(tile_cols), _ptr(out))
    return out


def ref_reduce_middle(x: np.ndarray, z: np.ndarray, lam: int, pad_k: int = 0) -> np.ndarray:
    d0, dk, dc = x.shape
    out = np.full((d0, dc), -12345.0, np.float32)
    ref().ref_reduce_middle(_ptr(x), _ptr(z), C.c_uint32(d0), C.c_uint32(dk), C.c_uint32(dc),
                            C.c_int(lam), C.c_uint32(pad_k), _ptr(out))
    return out


def ref_fold(v: np.ndarray, op: str, init: float, kind: str = "seq") -> float:
    v = np.ascontiguousarray(v, np.float32)
    return float(ref().ref_fold(_ptr(v), C.c_uint32(v.size), C.c_int({"sum": 0, "max": 1}[op]),
                                C.c_float(init), C.c_int({"seq": 0, "warp": 1}[kind])))
