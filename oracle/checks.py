"""Parity criteria shared by the tests, the smoke check and the benchmark's pre-timing check.

Test infrastructure only. The oracle folds sequentially in fp32, as the
reference's loops do; for long rows that fold is itself further than 1e-5 from
the exact value while the kernels' trees are not. A kernel output is therefore
accepted when it is within 1e-5 (relative) of the fp64 evaluation of the same
formula AND within 1e-5 of the oracle plus the oracle's own measured distance
to that fp64 value.
"""
from __future__ import annotations

import numpy as np

from . import binding as O


def softmax_f64(x: np.ndarray) -> np.ndarray:
    x64 = x.astype(np.float64)
    e = np.exp(x64 - x64.max(1, keepdims=True))
    return e / e.sum(1, keepdims=True)


def softmax_close(got: np.ndarray, x: np.ndarray, want: np.ndarray | None = None) -> bool:
    want = O.softmax_rows(x) if want is None else want
    f64 = softmax_f64(x)
    ok64 = (np.abs(got - f64) <= 1e-5 * f64 + 1e-37).all()
    oko = (np.abs(got - want) <= 1e-5 * want + np.abs(want - f64) + 1e-37).all()
    return bool(ok64 and oko)


def rowsum_close(got: np.ndarray, x: np.ndarray, a: float = 0.5, b: float = 0.25) -> bool:
    want = O.map_rowsum_affine_sq(x, a, b)
    f64 = O.map_rowsum_affine_sq_f64(x, a, b)
    return bool((np.abs(got - f64) <= 1e-5 * f64).all() and
                (np.abs(got - want) <= 1e-5 * np.abs(want) + np.abs(want - f64)).all())


def _bf16_ulp(v: np.ndarray) -> np.ndarray:
    return 2.0 ** (np.floor(np.log2(np.maximum(np.abs(v), 1e-38))) - 7)


def layernorm_bf16_close(got_bits, x_bits, g_bits, b_bits, eps: float = 1e-5, want_bits=None,
                         max_mismatch: float = 0.02) -> bool:
    """bf16 layer-norm outputs against the fp64 formula and against the oracle.

    y64 is the formula in fp64 on the same bf16 inputs, r64 its bf16 rounding. fp32err is the fp32
    error (1e-5 relative) of the two terms x_hat*gamma and beta, which matters only where they cancel
    to a value near zero, plus the error an fp32 mean leaves on x - mean (1e-6 of |mean| + std), which
    matters only for elements that sit on the mean.
      * the kernel must be a rounding of a value that close to exact: |got - y64| <= ulp/2 + fp32err;
      * against the oracle: |got - want| <= ulp + fp32err + |want - r64|, and the two may round
        differently only rarely: frac(got != want) <= max_mismatch + frac(want != r64).
    The |want - r64| terms are the oracle's own distance from the exact result: its sequential fp32
    variance fold drifts by a few 1e-5 on rows of 1e5 elements and more.
    """
    want_bits = O.layernorm_rows_bf16(x_bits, g_bits, b_bits, eps) if want_bits is None else want_bits
    got, want = O.bf16_to_f32(got_bits).astype(np.float64), O.bf16_to_f32(want_bits).astype(np.float64)
    x, g, b = (O.bf16_to_f32(t).astype(np.float64) for t in (x_bits, g_bits, b_bits))
    xhat = (x - x.mean(1, keepdims=True)) / np.sqrt(x.var(1, keepdims=True) + eps)
    y64 = xhat * g + b
    r64_bits = O.f32_to_bf16(y64.astype(np.float32))
    r64 = O.bf16_to_f32(r64_bits).astype(np.float64)
    # ... plus the floor any fp32 mean leaves on x - mean: a relative 1e-6 of (|mean| + std), scaled like x_hat
    std = np.sqrt(x.var(1, keepdims=True) + eps)
    fp32err = 1e-5 * (np.abs(xhat * g) + np.abs(b)) + 1e-6 * (np.abs(x.mean(1, keepdims=True)) / std + 1.0) * np.abs(g)
    ulp = _bf16_ulp(np.maximum(np.abs(y64), np.abs(got)))
    ok_exact = (np.abs(got - y64) <= 0.5 * ulp + fp32err + 1e-30).all()
    ok_oracle = (np.abs(got - want) <= _bf16_ulp(want) + fp32err + np.abs(want - r64)).all()
    ok_rate = (got_bits != want_bits).mean() <= max_mismatch + (want_bits != r64_bits).mean()
    return bool(ok_exact and ok_oracle and ok_rate)
