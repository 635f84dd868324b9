"""Parity criteria shared by the tests, the smoke check and the benchmark's pre-timing check.

Test infrastructure only. The oracle folds sequentially in fp32, as the
reference's loops do; for long rows that fold is itself further than 1e-5 from
the exact value while the kernels' trees are not. A kernel output is therefore
accepted when it is within 1e-5 (relative) of the fp64 evaluation of the same
formula AND within 1e-5 of the oracle plus the oracle's own measured distance
to that fp64 value.

Every criterion exists in two forms: `*_report` returns a Report that also counts
how many elements met the bare criterion "within 1e-5 relative of the oracle"
(one bf16 ulp for bf16 outputs) and how many passed only through the added
terms, so that the widening is visible wherever a check runs; `*_close` is
`report.ok`.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from . import binding as O


@dataclass
class Report:
    """Outcome of one parity check over `checked` elements.

    failed: elements outside the accepted criterion; via_fp64_term: elements that are accepted but
    differ from the ORACLE by more than the bare tolerance (1e-5 relative; one bf16 ulp for bf16
    outputs), i.e. that pass only because the oracle is charged its own distance to the fp64 value
    (or, for layer-norm, the fp32 floor of the terms that cancel)."""
    checked: int = 0
    failed: int = 0
    via_fp64_term: int = 0
    extra_ok: bool = True   # criteria that are not per element (e.g. the rate of differently rounded outputs)

    @property
    def ok(self) -> bool:
        return self.failed == 0 and self.extra_ok

    def merge(self, other: "Report") -> "Report":
        self.checked += other.checked
        self.failed += other.failed
        self.via_fp64_term += other.via_fp64_term
        self.extra_ok = self.extra_ok and other.extra_ok
        return self

    def as_dict(self) -> dict:
        return {"checked": int(self.checked), "failed": int(self.failed), "via_fp64_term": int(self.via_fp64_term)}


def _over_slabs(fn, starts):
    """fn(start) for every slab, a few at a time on threads (numpy and the oracle release the GIL)."""
    import os
    from concurrent.futures import ThreadPoolExecutor
    starts = list(starts)
    if len(starts) <= 1:
        return [fn(s) for s in starts]
    with ThreadPoolExecutor(max(1, min(len(starts), (os.cpu_count() or 2) // 2, 8))) as ex:
        return list(ex.map(fn, starts))


def _two_sided(got, want, f64, tiny=0.0) -> Report:
    """|got - f64| <= 1e-5 |f64| and |got - want| <= 1e-5 |want| + |want - f64|, per element."""
    d_o = np.abs(got - want)
    bare = d_o <= 1e-5 * np.abs(want) + tiny
    accepted = (np.abs(got - f64) <= 1e-5 * np.abs(f64) + tiny) & (d_o <= 1e-5 * np.abs(want) + np.abs(want - f64) + tiny)
    return Report(checked=got.size, failed=int((~accepted).sum()), via_fp64_term=int((accepted & ~bare).sum()))


def softmax_f64(x: np.ndarray) -> np.ndarray:
    x64 = x.astype(np.float64)
    e = np.exp(x64 - x64.max(1, keepdims=True))
    return e / e.sum(1, keepdims=True)


def softmax_report(got: np.ndarray, x: np.ndarray, want: np.ndarray | None = None, slab: int = 2048) -> Report:
    """Row softmax against the oracle and the fp64 formula, in slabs of rows (bounded temporaries)."""
    def one(lo):
        xs = x[lo:lo + slab]
        ws = O.softmax_rows(xs) if want is None else want[lo:lo + slab]
        return _two_sided(got[lo:lo + slab], ws, softmax_f64(xs), tiny=1e-37)

    rep = Report()
    for r in _over_slabs(one, range(0, x.shape[0], slab)):
        rep.merge(r)
    return rep


def softmax_report_fast(got: np.ndarray, x: np.ndarray, want: np.ndarray | None = None) -> Report:
    """softmax_report with the per-element rule evaluated by the C checker (whole tensors in seconds)."""
    got, x = np.ascontiguousarray(got), np.ascontiguousarray(x)
    want = O.softmax_rows(x) if want is None else np.ascontiguousarray(want)
    c = O.check_softmax(got, want, x).sum(0)
    return Report(checked=int(c[0]), failed=int(c[1]), via_fp64_term=int(c[2]))


def softmax_close(got: np.ndarray, x: np.ndarray, want: np.ndarray | None = None) -> bool:
    return softmax_report(got, x, want).ok


def rowsum_report(got: np.ndarray, x: np.ndarray, a: float = 0.5, b: float = 0.25) -> Report:
    want = O.map_rowsum_affine_sq(x, a, b)
    f64 = O.map_rowsum_affine_sq_f64(x, a, b)
    return _two_sided(got, want, f64)


def rowsum_close(got: np.ndarray, x: np.ndarray, a: float = 0.5, b: float = 0.25) -> bool:
    return rowsum_report(got, x, a, b).ok


def outer_sum_report(got: np.ndarray, want: np.ndarray, t: np.ndarray) -> Report:
    """Sums over axis 1 of t[b, k, c] whose terms cancel: per element against 1e-5 * sum_k |t|.

    The bare criterion (1e-5 of the oracle's value) has no meaning for a sum that cancels to nearly
    zero; the elements that need the sum-of-magnitudes denominator are counted as via_fp64_term."""
    d = np.abs(got - want)
    mag = np.abs(t).sum(1, dtype=np.float64)
    accepted = d <= 1e-5 * mag
    bare = d <= 1e-5 * np.abs(want)
    return Report(checked=got.size, failed=int((~accepted).sum()), via_fp64_term=int((accepted & ~bare).sum()))


def _bf16_ulp(v: np.ndarray) -> np.ndarray:
    """2 ** (floor(log2 |v|) - 7): the spacing of bf16 values (8 significant bits) at |v|."""
    _, e = np.frexp(np.maximum(np.abs(v), 1e-38))   # |v| = m * 2**e with m in [0.5, 1)
    return np.ldexp(1.0, e - 8)


def layernorm_bf16_report(got_bits, x_bits, g_bits, b_bits, eps: float = 1e-5, want_bits=None,
                          max_mismatch: float = 0.02, slab: int = 2048) -> Report:
    """bf16 layer-norm outputs against the fp64 formula and against the oracle.

    y64 is the formula in fp64 on the same bf16 inputs, r64 its bf16 rounding. fp32err is the fp32
    error (1e-5 relative) of the two terms x_hat*gamma and beta, which matters only where they cancel
    to a value near zero, plus the error an fp32 mean leaves on x - mean (1e-6 of |mean| + std), which
    matters only for elements that sit on the mean.
      * the kernel must be a rounding of a value that close to exact: |got - y64| <= ulp/2 + fp32err;
      * against the oracle: |got - want| <= ulp + fp32err + |want - r64|, and the two may round
        differently only rarely: frac(got != want) <= max_mismatch + frac(want != r64).
    The |want - r64| terms are the oracle's own distance from the exact result: its sequential fp32
    variance fold drifts by a few 1e-5 on rows of 1e5 elements and more. The bare criterion counted in
    via_fp64_term is |got - want| <= one bf16 ulp of want. Rows are processed in slabs.
    """
    g, b = (O.bf16_to_f32(t).astype(np.float64) for t in (g_bits, b_bits))

    def one(lo):
        xb = x_bits[lo:lo + slab]
        gb = got_bits[lo:lo + slab]
        wb = O.layernorm_rows_bf16(xb, g_bits, b_bits, eps) if want_bits is None else want_bits[lo:lo + slab]
        got, want = O.bf16_to_f32(gb).astype(np.float64), O.bf16_to_f32(wb).astype(np.float64)
        x = O.bf16_to_f32(xb).astype(np.float64)
        mean, var = x.mean(1, keepdims=True), x.var(1, keepdims=True)
        std = np.sqrt(var + eps)
        xhat = (x - mean) / std
        y64 = xhat * g + b
        r64_bits = O.f32_to_bf16(y64.astype(np.float32))
        r64 = O.bf16_to_f32(r64_bits).astype(np.float64)
        # ... plus the floor any fp32 mean leaves on x - mean: a relative 1e-6 of (|mean| + std), scaled like x_hat
        fp32err = 1e-5 * (np.abs(xhat * g) + np.abs(b)) + 1e-6 * (np.abs(mean) / std + 1.0) * np.abs(g)
        ulp = _bf16_ulp(np.maximum(np.abs(y64), np.abs(got)))
        d_o = np.abs(got - want)
        accepted = (np.abs(got - y64) <= 0.5 * ulp + fp32err + 1e-30) & \
                   (d_o <= _bf16_ulp(want) + fp32err + np.abs(want - r64))
        bare = d_o <= _bf16_ulp(want)
        return (Report(checked=got.size, failed=int((~accepted).sum()), via_fp64_term=int((accepted & ~bare).sum())),
                int((gb != wb).sum()), int((wb != r64_bits).sum()))

    rep, differ, oracle_off = Report(), 0, 0
    for r, d, o in _over_slabs(one, range(0, x_bits.shape[0], slab)):
        rep.merge(r)
        differ += d
        oracle_off += o
    n = max(rep.checked, 1)
    rep.extra_ok = differ / n <= max_mismatch + oracle_off / n
    return rep


def layernorm_bf16_report_fast(got_bits, x_bits, g_bits, b_bits, eps: float = 1e-5, want_bits=None,
                               max_mismatch: float = 0.02) -> Report:
    """layernorm_bf16_report with the per-element rule evaluated by the C checker."""
    got_bits, x_bits = np.ascontiguousarray(got_bits), np.ascontiguousarray(x_bits)
    want_bits = O.layernorm_rows_bf16(x_bits, g_bits, b_bits, eps) if want_bits is None else np.ascontiguousarray(want_bits)
    c = O.check_layernorm_bf16(got_bits, want_bits, x_bits, g_bits, b_bits, eps).sum(0)
    n = max(int(c[0]), 1)
    return Report(checked=int(c[0]), failed=int(c[1]), via_fp64_term=int(c[2]),
                  extra_ok=bool(int(c[3]) / n <= max_mismatch + int(c[4]) / n))


def layernorm_bf16_close(got_bits, x_bits, g_bits, b_bits, eps: float = 1e-5, want_bits=None,
                         max_mismatch: float = 0.02) -> bool:
    return layernorm_bf16_report(got_bits, x_bits, g_bits, b_bits, eps, want_bits, max_mismatch).ok
