"""The map-only operator (tcab_map) and the typed lambda vocabulary on a B200, through the C ABI.

Oracle: the caller's expression text compiled by the host C++ compiler and run element by element
(oracle/lambda_eval.py) -- what the reference does with a lambda, on the CPU
(internal/cg/cxx/expr.go:14-101 prints it, the C++ compiler gives it its meaning).
Tolerances, as stated for this path: integer, index and bool-selected outputs bit-exact; fp32 maps
within 2 ulp. For the math builtins the 2 ulp are measured against the correctly rounded fp64 value
(the way CUDA states its own bounds); for plain arithmetic against the host evaluation, where the
only admissible difference is one FMA contraction per operation (design/syntax-design.md:601-607).
"""
import numpy as np
import pytest
import torch

import tcacomp_b200 as T
from guards import guarded_input

pytestmark = pytest.mark.gpu

NP2T = {np.dtype(np.float32): torch.float32, np.dtype(np.int32): torch.int32, np.dtype(np.uint32): torch.uint32}


def to_dev(a, dev):
    """numpy -> device; uint16 arrays are bf16 bit patterns."""
    return guarded_input(a, dev)       # inside NaN / wild-integer bands: a read outside the operand cannot pass by luck


def to_host(t):
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).cpu().numpy().view(np.uint16)
    if t.dtype == torch.uint32:
        return t.view(torch.int32).cpu().numpy().view(np.uint32)
    return t.cpu().numpy()


def torch_dtype(np_dtype):
    return torch.bfloat16 if np.dtype(np_dtype) == np.uint16 else NP2T[np.dtype(np_dtype)]


def ulp_distance(a, b):
    """Distance in units in the last place between two float32 arrays (monotone integer images of the floats)."""
    def key(x):
        i = x.astype(np.float32).view(np.int32).astype(np.int64)
        return np.where(i < 0, -(i & 0x7fffffff), i)
    return np.abs(key(a) - key(b))


def run_map(expr, arrays, dev, out_np_dtype, captures=()):
    from oracle import lambda_eval
    want = lambda_eval.evaluate(expr, arrays, captures, out_np_dtype)
    got = to_host(T.map([to_dev(a, dev) for a in arrays], expr, captures=captures, out_dtype=torch_dtype(out_np_dtype)))
    return got, want


def inputs(rng, n, kind):
    if kind == "f":
        return rng.uniform(-4, 4, n).astype(np.float32)
    if kind == "i":
        return rng.integers(-1000, 1000, n).astype(np.int32)
    if kind == "u":
        return rng.integers(0, 1 << 20, n).astype(np.uint32)
    from oracle import binding as O
    return O.f32_to_bf16(rng.uniform(-4, 4, n).astype(np.float32))


# One case per operator of the reference's vocabulary (pkg/expr.go:185-203, 271; internal/cg/cxx/naming.go:126-183).
# (expression, operand kinds, output dtype): every one of these is exact arithmetic or a selection, so bit-exact.
EXACT = [
    ("p0 > p1 ? p0 : p1", "ff", np.float32), ("p0 >= 0.0f ? p0 : 0.0f", "f", np.float32),
    ("p0 < p1 ? 1 : 0", "ff", np.int32), ("p0 <= p1 ? 1 : 0", "ii", np.int32),
    ("p0 == p1 ? 7u : 9u", "uu", np.uint32), ("p0 != 3 ? p0 : -p0", "i", np.int32),
    ("(p0 > 0.0f && p1 > 0.0f) ? 1 : 0", "ff", np.int32), ("(p0 > 0.0f || p1 > 0.0f) ? 1 : 0", "ff", np.int32),
    ("!(p0 > p1) ? p0 : p1", "ff", np.float32),
    ("p0 % 7", "i", np.int32), ("p0 % 7u", "u", np.uint32), ("p0 / 3", "i", np.int32),
    ("p0 & p1", "ii", np.int32), ("p0 | p1", "uu", np.uint32), ("p0 ^ p1", "ii", np.int32), ("~p0", "u", np.uint32),
    ("p0 << 3", "i", np.int32), ("p0 >> 2", "i", np.int32), ("p0 >> 5u", "u", np.uint32),
    ("p0 + p1", "ii", np.int32), ("p0 - p1", "uu", np.uint32), ("p0 * p1", "ii", np.int32), ("-p0", "f", np.float32),
    ("umin(p0, p1) + umax(p0, 77u)", "uu", np.uint32),
    ("f32(p0)", "i", np.float32), ("f32(p0)", "u", np.float32), ("f32(p0)", "b", np.float32),
    ("i32(p0)", "f", np.int32), ("u32(fabsf(p0))", "f", np.uint32), ("bf16(p0)", "f", np.uint16),
    ("i32(p0)", "b", np.int32), ("bf16(p0)", "i", np.uint16), ("u32(p0)", "i", np.uint32),
    ("static_cast<int32_t>(p0) + static_cast<int32_t>(static_cast<float>(p1))", "fb", np.int32),
    ("p0 + p1", "ff", np.float32), ("p0 * p1", "ff", np.float32), ("p0 / p1", "ff", np.float32), ("p0 - 1.5f", "f", np.float32),
    ("fminf(p0, p1)", "ff", np.float32), ("fmaxf(p0, 0.0f)", "f", np.float32), ("fabsf(p0)", "f", np.float32),
    ("sqrtf(fabsf(p0))", "f", np.float32), ("fmaf(p0, p1, p2)", "fff", np.float32),
    ("f32(p0) > 0.0f ? p0 : p1", "bb", np.uint16),                     # a bf16 value can be selected as it is
    ("bf16(fmaxf(f32(p0) + f32(p1), 0.0f))", "bb", np.uint16),
]


@pytest.mark.parametrize("expr,kinds,out_dtype", EXACT)
def test_operator_is_bit_exact(cuda, expr, kinds, out_dtype):
    rng = np.random.default_rng(len(expr) * 7 + len(kinds))
    arrays = [inputs(rng, 5003, k) for k in kinds]    # 5003: full groups of eight and a ragged end
    got, want = run_map(expr, arrays, cuda, out_dtype)
    assert np.array_equal(got, want), expr


def test_arithmetic_within_one_contraction_of_the_host(cuda):
    # a product feeding a sum may be contracted into one fused multiply-add on the device (permitted per
    # operation); the host evaluates with two roundings. 2 ulp of the result bounds the difference when
    # the sum does not cancel (all terms positive here).
    rng = np.random.default_rng(3)
    x, y = rng.uniform(0.5, 4, 100003).astype(np.float32), rng.uniform(0.5, 4, 100003).astype(np.float32)
    got, want = run_map("(0.5f * p0 + 0.25f) * (0.5f * p0 + 0.25f) + p1 * p1", [x, y], cuda, np.float32)
    assert ulp_distance(got, want).max() <= 2
    got, want = run_map("c0 * p0 + c1 * p1", [x, y], cuda, np.float32, captures=(1.25, 0.75))
    assert ulp_distance(got, want).max() <= 2


BUILTINS = {
    # name: (device expression, fp64 formula, operand ranges)
    "expf": ("expf(p0)", lambda a: np.exp(a), [(-87.0, 88.0)]),
    "logf": ("logf(p0)", lambda a: np.log(a), [(1e-30, 1e30)]),
    "sqrtf": ("sqrtf(p0)", lambda a: np.sqrt(a), [(1e-30, 1e30)]),
    "rsqrtf": ("rsqrtf(p0)", lambda a: 1.0 / np.sqrt(a), [(1e-30, 1e30)]),
    "fabsf": ("fabsf(p0)", lambda a: np.abs(a), [(-1e30, 1e30)]),
    "tanhf": ("tanhf(p0)", lambda a: np.tanh(a), [(-12.0, 12.0)]),
    "sinf": ("sinf(p0)", lambda a: np.sin(a), [(-100.0, 100.0)]),
    "cosf": ("cosf(p0)", lambda a: np.cos(a), [(-100.0, 100.0)]),
    "fminf": ("fminf(p0, p1)", lambda a, b: np.minimum(a, b), [(-5.0, 5.0), (-5.0, 5.0)]),
    "fmaxf": ("fmaxf(p0, p1)", lambda a, b: np.maximum(a, b), [(-5.0, 5.0), (-5.0, 5.0)]),
    "fmaf": ("fmaf(p0, p1, p2)", lambda a, b, c: a * b + c, [(-5.0, 5.0), (-5.0, 5.0), (-5.0, 5.0)]),
}


@pytest.mark.parametrize("name", sorted(BUILTINS))
def test_fp32_map_within_2_ulp_of_fp64(cuda, name):
    """fp32 maps: within 2 ulp -- every builtin of the vocabulary (internal/ir/builtins.go:25-39) through the
    map-only path, against the fp64 value of the same formula rounded to fp32."""
    expr, f64, ranges = BUILTINS[name]
    rng = np.random.default_rng(sum(map(ord, name)))
    n = 1 << 20
    arrays = []
    for lo, hi in ranges:
        if lo > 0 and hi / lo > 1e6:   # wide positive ranges: uniform in the exponent
            arrays.append(np.exp(rng.uniform(np.log(lo), np.log(hi), n)).astype(np.float32))
        else:
            arrays.append(rng.uniform(lo, hi, n).astype(np.float32))
    got = to_host(T.map([to_dev(a, cuda) for a in arrays], expr))
    want = f64(*[a.astype(np.float64) for a in arrays]).astype(np.float32)
    d = ulp_distance(got, want)
    assert d.max() <= 2, (name, int(d.max()), arrays[0][int(d.argmax())])


@pytest.mark.parametrize("shape", [(0,), (1,), (7,), (8,), (9,), (3, 5), (2, 3, 5, 7), (1025, 33), (64, 4096)])
def test_shapes_ragged_ends_and_guard_bands(cuda, shape):
    rng = np.random.default_rng(int(np.prod(shape)) + len(shape))
    n = int(np.prod(shape))
    x = rng.uniform(-3, 3, shape).astype(np.float32)
    guard, canary = 64, -12345.0
    buf = torch.full((n + 2 * guard,), canary, device=cuda)
    out = buf[guard:guard + n].view(*shape)
    T.map([to_dev(x, cuda)], "p0 * 2.0f - 1.0f", out=out)
    b = buf.cpu().numpy()
    assert (b[:guard] == canary).all() and (b[guard + n:] == canary).all(), "the kernel wrote outside its output"
    want = x * np.float32(2.0) - np.float32(1.0)   # exact in fp32 with or without contraction (scaling by 2)
    assert np.array_equal(b[guard:guard + n].reshape(shape), want)


def test_pointers_aligned_to_their_element_only(cuda):
    # operands that start 4 (2) bytes into a 16-byte vector take the single-element kernel
    rng = np.random.default_rng(5)
    n = 4099
    x = rng.uniform(-3, 3, n).astype(np.float32)
    base = torch.zeros(n + 1, device=cuda)
    xd = base[1:]
    xd.copy_(to_dev(x, cuda))
    assert xd.data_ptr() % 16 == 4
    got = T.map([xd], "fmaxf(p0, 0.0f)").cpu().numpy()
    assert np.array_equal(got, np.maximum(x, 0))
    from oracle import binding as O
    hb = O.f32_to_bf16(x)
    bb = torch.zeros(n + 1, device=cuda, dtype=torch.bfloat16)
    bd = bb[1:]
    bd.copy_(to_dev(hb, cuda))
    assert bd.data_ptr() % 16 == 2
    got = T.map([bd], "f32(p0) * 0.5f", out_dtype=torch.float32).cpu().numpy()
    assert np.array_equal(got, O.bf16_to_f32(hb) * np.float32(0.5))


def test_ahead_of_time_and_compiled_lambdas_agree(cuda):
    # "(p0 * c0) + c1" has an ahead-of-time kernel; the same arithmetic spelled with an extra exact step does not
    rng = np.random.default_rng(6)
    x = rng.uniform(-3, 3, (257, 129)).astype(np.float32)
    xd = to_dev(x, cuda)
    n0 = T.launch_count()
    a = T.map([xd], "p0 * 3.0f + 0.5f").cpu().numpy()
    b = T.map([xd], "(p0 * 3.0f + 0.5f) * 1.0f").cpu().numpy()
    assert T.launch_count() - n0 == 2
    assert ulp_distance(a, b).max() <= 1


def test_type_errors_reach_the_caller(cuda):
    x = torch.zeros((4, 4), device=cuda)
    with pytest.raises(T.TcabError) as e:
        T.map([x], "p0", out_dtype=torch.bfloat16)          # the store never converts
    assert e.value.status == T._lib.ERR_DTYPE and "convert explicitly" in e.value.message
    with pytest.raises(T.TcabError) as e:
        T.map([x], "p0 * 2")                                 # f32 * i32
    assert e.value.status == T._lib.ERR_INVALID_ARG and "operand types differ" in e.value.message
    with pytest.raises(T.TcabError) as e:
        T.map([x, torch.zeros((4, 5), device=cuda)], "p0 + p1")
    assert e.value.status == T._lib.ERR_SHAPE


# ----------------------------------------------------------------------------
# typed operands inside reductions and contractions
# ----------------------------------------------------------------------------
@pytest.mark.parametrize("shape,axis", [((37, 1000), 1), ((5, 300, 132), 1), ((3, 64), 1), ((2, 70000), 1), ((6, 50, 7), 1)])
def test_reduction_over_bf16_and_integer_operands(cuda, shape, axis):
    from oracle import binding as O
    rng = np.random.default_rng(shape[-1])
    xb = O.f32_to_bf16(rng.uniform(-1, 1, shape).astype(np.float32))
    w = rng.uniform(-1, 1, shape).astype(np.float32)
    k = rng.integers(0, 9, shape).astype(np.int32)
    ax = axis if len(shape) == 3 else len(shape) - 1
    got = T.chain_reduce([to_dev(xb, cuda), to_dev(w, cuda), to_dev(k, cuda)],
                         "f32(p0) * p1 * (p2 % 3 == 0 ? 2.0f : 0.5f)", axis=ax).cpu().numpy()
    terms = O.bf16_to_f32(xb).astype(np.float64) * w * np.where(k % 3 == 0, 2.0, 0.5)
    assert (np.abs(got - terms.sum(ax)) <= 1e-5 * np.abs(terms).sum(ax) + 1e-30).all()
    # max over a bf16 operand: order-independent, bit-exact
    got = T.chain_reduce([to_dev(xb, cuda)], "f32(p0)", combine_expr="fmaxf(p0, p1)", init=-np.inf, axis=ax).cpu().numpy()
    assert np.array_equal(got, O.bf16_to_f32(xb).max(ax))


@pytest.mark.parametrize("m,k,n,nk", [(128, 64, 192, True), (70, 100, 36, False), (256, 512, 256, False), (33, 7, 5, True)])
def test_contraction_over_bf16_operands(cuda, m, k, n, nk):
    # testing/kernels/llm/qk_score.tca with bf16 storage: scores[m,n] = scale * sum_k q[m,k] * key[n,k], f32 accumulate
    from oracle import binding as O
    rng = np.random.default_rng(m + k + n)
    q = O.f32_to_bf16(rng.uniform(-1, 1, (m, k)).astype(np.float32))
    key = O.f32_to_bf16(rng.uniform(-1, 1, (n, k) if nk else (k, n)).astype(np.float32))
    got = T.chain_contract(to_dev(q, cuda), to_dev(key, cuda), "f32(p0) * f32(p1)", rhs_is_nk=nk,
                           post_expr="p0 * c0", captures=(0.125,)).cpu().numpy()
    qf, kf = O.bf16_to_f32(q).astype(np.float64), O.bf16_to_f32(key).astype(np.float64)
    want = 0.125 * (qf @ (kf.T if nk else kf))
    mag = 0.125 * (np.abs(qf) @ np.abs(kf.T if nk else kf))
    assert (np.abs(got - want) <= 1e-5 * mag + 1e-30).all()
    # mixed: bf16 lhs, f32 rhs
    kf32 = rng.uniform(-1, 1, (n, k) if nk else (k, n)).astype(np.float32)
    got = T.chain_contract(to_dev(q, cuda), to_dev(kf32, cuda), "f32(p0) * p1", rhs_is_nk=nk).cpu().numpy()
    want = qf @ (kf32.astype(np.float64).T if nk else kf32.astype(np.float64))
    mag = np.abs(qf) @ np.abs(kf32.astype(np.float64).T if nk else kf32.astype(np.float64))
    assert (np.abs(got - want) <= 1e-5 * mag + 1e-30).all()


@pytest.mark.parametrize("m,k,n,nk", [(300, 264, 520, False), (300, 264, 516, True), (1, 8, 8, False), (129, 4096, 264, True),
                                      (513, 72, 1032, False), (2048, 2048, 2048, False), (700, 1024, 260, True),
                                      (100, 8192, 520, False), (260, 2048, 1028, True), (128, 1024, 256, False)])
def test_bf16_product_chains_run_on_the_tensor_cores(cuda, m, k, n, nk):
    # map = the plain product of two bf16 operands, sum reducer, init 0, stored as it is or scaled: the library takes
    # the tcgen05 kernel with fp32 accumulation and an fp32 store (one launch). Products of bf16 values are exact in
    # fp32, so only the order of the sum differs from the scalar kernel (tuning value gemm p2 = 64 keeps that one).
    from oracle import binding as O
    rng = np.random.default_rng(m + k + n)
    a = O.f32_to_bf16(rng.uniform(-1, 1, (m, k)).astype(np.float32))
    b = O.f32_to_bf16(rng.uniform(-1, 1, (n, k) if nk else (k, n)).astype(np.float32))
    af, bf = O.bf16_to_f32(a).astype(np.float64), O.bf16_to_f32(b).astype(np.float64)
    bm = bf.T if nk else bf
    want, mag = af @ bm, np.abs(af) @ np.abs(bm)
    for post, caps, scale in ((None, (), 1.0), ("p0 * c0", (0.125,), 0.125), ("0.5f * p0", (), 0.5)):
        out = torch.full((m + 2, n), -7.0, device=cuda)             # canary rows around the output
        n0 = T.launch_count()
        T.chain_contract(to_dev(a, cuda), to_dev(b, cuda), "f32(p0) * f32(p1)", rhs_is_nk=nk, post_expr=post, captures=caps,
                         out=out[1:m + 1])
        assert T.launch_count() - n0 == 1
        got = out.cpu().numpy()
        assert (got[0] == -7.0).all() and (got[-1] == -7.0).all()
        assert (np.abs(got[1:-1] - scale * want) <= 1e-5 * scale * mag + 1e-30).all()
    try:    # the scalar kernel on the same operands: the same sums in another order
        T.tune("gemm", 0, 0, 64)
        ref = T.chain_contract(to_dev(a, cuda), to_dev(b, cuda), "f32(p0) * f32(p1)", rhs_is_nk=nk).cpu().numpy()
    finally:
        T.tune("gemm")
    tc = T.chain_contract(to_dev(a, cuda), to_dev(b, cuda), "f32(p0) * f32(p1)", rhs_is_nk=nk).cpu().numpy()
    assert (np.abs(tc - ref) <= 2e-5 * mag + 1e-30).all()
    # anything else keeps the scalar kernel: another map, another reducer, rows that are not 16-byte multiples
    got = T.chain_contract(to_dev(a, cuda), to_dev(b, cuda), "f32(p0) * f32(p1) + 1.0f", rhs_is_nk=nk).cpu().numpy()
    assert (np.abs(got - (want + k)) <= 1e-5 * (mag + k) + 1e-30).all()


@pytest.mark.parametrize("m,k,n,nk", [(2048, 512, 2048, False), (2048, 260, 2056, True), (4100, 256, 1032, False),
                                      (1024, 1024, 1024, False), (520, 2048, 1028, True)])
def test_large_f32_product_chains_run_on_the_tensor_cores(cuda, m, k, n, nk):
    # fp32 operands, the plain product, a sum from 0: from 64 output tiles of 256 x 256 on, each operand is cut into
    # three bf16 pieces and the six significant piece products run as one bf16 contraction over 6 K (three launches).
    # What is dropped is below 3 * 2^-24 of |a b| per product; small problems keep the scalar kernel and with it the
    # reference's ascending order over k (tuning value gemm p2 = 64 keeps it for every size).
    rng = np.random.default_rng(m + k + n)
    a = rng.normal(0, 1, (m, k)).astype(np.float32)
    b = rng.normal(0, 1, (n, k) if nk else (k, n)).astype(np.float32)
    a[0, :8] = [1e-30, -1e30, 3.0, 1e-38, 0.0, -0.0, 65504.0, 1.0000001]      # tiny, huge and exact values
    ad, bd = to_dev(a, cuda), to_dev(b, cuda)
    a64, b64 = a.astype(np.float64), b.astype(np.float64)
    bm = b64.T if nk else b64
    want, mag = a64 @ bm, np.abs(a64) @ np.abs(bm)
    out = torch.full((m + 2, n), -7.0, device=cuda)
    n0 = T.launch_count()
    T.chain_contract(ad, bd, rhs_is_nk=nk, post_expr="p0 * c0", captures=(0.5,), out=out[1:m + 1])
    assert T.launch_count() - n0 == 3
    got = out.cpu().numpy()
    assert (got[0] == -7.0).all() and (got[-1] == -7.0).all()
    err = np.abs(got[1:-1] - 0.5 * want) / (0.5 * mag)
    assert err.max() <= 2e-6, err.max()                 # the scalar kernel's bound on the same data is 1e-5
    try:
        T.tune("gemm", 0, 0, 64)
        n0 = T.launch_count()
        ref = T.chain_contract(ad, bd, rhs_is_nk=nk).cpu().numpy()
        assert T.launch_count() - n0 == 1
    finally:
        T.tune("gemm")
    tc = T.chain_contract(ad, bd, rhs_is_nk=nk).cpu().numpy()
    assert (np.abs(tc - ref) <= 4e-6 * mag).all()
    # a reducer other than the sum, or an init other than 0, keeps the scalar kernel
    n0 = T.launch_count()
    T.chain_contract(ad, bd, rhs_is_nk=nk, init=1.0)
    assert T.launch_count() - n0 == 1
    # a workspace too small for all pieces at once: blocks of rows of a against blocks of columns of b (the K ranges
    # of a block product may be cut differently over CTAs: the same sums in another order)
    try:
        T.tune("gemm", 0, 0, 128, max(8, (2304 * k * 12 >> 20) + 1))     # room for 1024 + 1024 (+ 256) lines
        out = torch.full((m + 2, n), -7.0, device=cuda)
        n0 = T.launch_count()
        T.chain_contract(ad, bd, rhs_is_nk=nk, out=out[1:m + 1])
        assert T.launch_count() - n0 > 3 or m + n <= 2304
    finally:
        T.tune("gemm")
    got = out.cpu().numpy()
    assert (got[0] == -7.0).all() and (got[-1] == -7.0).all()
    assert (np.abs(got[1:-1] - tc) <= 1e-6 * mag).all()


# ----------------------------------------------------------------------------
# operands that bind a subset of the iteration axes: one value per row, one row shared by all rows
# ----------------------------------------------------------------------------
def bcast(a, shape):
    return np.ascontiguousarray(np.broadcast_to(a, shape))


@pytest.mark.parametrize("rows,cols", [(37, 1000), (5, 8), (300, 4096), (3, 13), (64, 20000), (41, 1001), (90, 3), (77, 1)])
def test_softmax_statement_by_statement_reads_row_values(oracle, cuda, rows, cols):
    """The softmax chain as the reference would have to spell it (pkg/local_test.go:17-68: a reduction stores into
    a rank-1 Local, the next statement reads it as x[i] inside the (i, j) iteration): m = max_j x; s = sum_j
    exp(x - m[i]); y = exp(x - m[i]) / s[i]. Three launches; against the one-launch operator and the oracle."""
    from oracle import checks, lambda_eval
    rng = np.random.default_rng(rows + cols)
    x = (4 * rng.normal(0, 1, (rows, cols))).astype(np.float32)
    xd = to_dev(x, cuda)
    m = T.chain_reduce([xd], "p0", combine_expr="fmaxf(p0, p1)", init=-np.inf)            # [rows]
    s = T.chain_reduce([xd, m.view(rows, 1)], "expf(p0 - p1)")                            # reads m[i]
    y = T.map([xd, m.view(rows, 1), s.view(rows, 1)], "expf(p0 - p1) / p2")
    assert np.array_equal(m.cpu().numpy(), x.max(1))
    mh = x.max(1, keepdims=True)
    want_s = np.exp(x.astype(np.float64) - mh).sum(1)
    assert (np.abs(s.cpu().numpy() - want_s) <= 1e-5 * want_s).all()
    assert checks.softmax_close(y.cpu().numpy(), x)
    # the map alone against the same expression in fp64 on the same row values: expf within 2 ulp and one
    # correctly rounded division
    sh = s.cpu().numpy().reshape(rows, 1)
    want = (np.exp((x - mh).astype(np.float64)) / sh.astype(np.float64)).astype(np.float32)
    assert ulp_distance(y.cpu().numpy(), want).max() <= 3
    # and, where the host's libm agrees with the device's expf, bit for bit against the host evaluation of the text
    host = lambda_eval.evaluate("expf(p0 - p1) / p2", [x, bcast(mh, x.shape), bcast(sh, x.shape)])
    assert ulp_distance(y.cpu().numpy(), host).max() <= 4 and (y.cpu().numpy() == host).mean() > 0.5


@pytest.mark.parametrize("rows,cols", [(33, 1024), (7, 10), (128, 8192), (19, 1003), (110, 5)])
def test_shared_rows_bias_and_layernorm_tail(oracle, cuda, rows, cols):
    from oracle import binding as O, lambda_eval
    rng = np.random.default_rng(rows * cols)
    x = rng.normal(0, 1, (rows, cols)).astype(np.float32)
    bias = rng.normal(0, 1, (1, cols)).astype(np.float32)
    got = T.map([to_dev(x, cuda), to_dev(bias, cuda)], "fmaxf(p0 + p1, 0.0f)").cpu().numpy()
    assert np.array_equal(got, np.maximum(x + bias, 0))
    # layer-norm's last map on bf16 rows: y = bf16((f32(x) - mean[i]) * rstd[i] * f32(gamma[j]) + f32(beta[j]))
    xb = O.f32_to_bf16(x)
    g = O.f32_to_bf16(rng.normal(1, 0.1, (1, cols)).astype(np.float32))
    b = O.f32_to_bf16(rng.normal(0, 0.1, (1, cols)).astype(np.float32))
    xf = O.bf16_to_f32(xb)
    mean = xf.mean(1, keepdims=True).astype(np.float32)
    rstd = (1.0 / np.sqrt(xf.var(1, keepdims=True) + 1e-5)).astype(np.float32)
    expr = "bf16((f32(p0) - p1) * p2 * f32(p3) + f32(p4))"
    with pytest.raises(ValueError):
        T.map([to_dev(xb, cuda)] * 7, expr)                    # at most six operands per lambda
    got = to_host(T.map([to_dev(xb, cuda), to_dev(mean, cuda), to_dev(rstd, cuda), to_dev(g, cuda), to_dev(b, cuda)], expr,
                        out_dtype=torch.bfloat16))
    want = lambda_eval.evaluate(expr, [xb, bcast(mean, x.shape), bcast(rstd, x.shape), bcast(g, x.shape), bcast(b, x.shape)],
                                out_dtype=np.uint16)
    # fused multiply-adds may differ from the host's separate roundings before the bf16 rounding: one bf16 ulp at
    # most, and rarely
    gf, wf = O.bf16_to_f32(got).astype(np.float64), O.bf16_to_f32(want).astype(np.float64)
    assert (np.abs(gf - wf) <= 2.0 ** -7 * np.maximum(np.abs(wf), 2.0 ** -10)).all()
    assert (got != want).mean() < 0.01
    # a reduction over a row weighted by a shared row: sum_j x[i][j] * w[j]
    got = T.chain_reduce([to_dev(x, cuda), to_dev(bias, cuda)], "p0 * p1").cpu().numpy()
    want = (x.astype(np.float64) * bias).sum(1)
    assert (np.abs(got - want) <= 1e-5 * np.abs(x.astype(np.float64) * bias).sum(1)).all()


def test_broadcast_shapes_are_checked(cuda):
    x = torch.zeros((6, 16), device=cuda)
    with pytest.raises(T.TcabError) as e:
        T.map([x, torch.zeros((6, 2), device=cuda)], "p0 + p1")
    assert e.value.status == T._lib.ERR_SHAPE
    with pytest.raises(T.TcabError) as e:     # a value per row needs the innermost axis to be the reduced one
        T.chain_reduce([torch.zeros((4, 6, 16), device=cuda), torch.zeros((4, 6, 1), device=cuda)], "p0 * p1", axis=1)
    assert e.value.status == T._lib.ERR_SHAPE


@pytest.mark.parametrize("nb,nk,nc", [(5, 300, 132), (2, 9, 7), (1, 5000, 64), (16, 8, 256), (3000, 40, 8), (700, 6, 512),
                                      (5000, 3, 4)])
def test_middle_axis_reduction_reads_a_value_per_output_cell(cuda, nb, nk, nc):
    """The reference's softmax suite kernel reduces over the MIDDLE axis (testing/kernels/fusion/softmax.tca). Written
    statement by statement its second reduction reads the first one's result m[i][j] inside the (i, k, j) iteration:
    an operand that lacks the reduced axis, one value per output cell."""
    rng = np.random.default_rng(nb + nk + nc)
    x = (3 * rng.normal(0, 1, (nb, nk, nc))).astype(np.float32)
    z = rng.uniform(0, 1, (nb, nk, nc)).astype(np.float32)
    xd, zd = to_dev(x, cuda), to_dev(z, cuda)
    m = T.chain_reduce([xd], "p0", combine_expr="fmaxf(p0, p1)", init=-np.inf, axis=1)                # [nb, nc]
    s = T.chain_reduce([xd, m.view(nb, 1, nc), zd], "expf(p0 - p1) * p2", axis=1).cpu().numpy()
    assert np.array_equal(m.cpu().numpy(), x.max(1))
    want = (np.exp(x.astype(np.float64) - x.max(1, keepdims=True)) * z).sum(1)
    assert (np.abs(s - want) <= 1e-5 * want + 1e-30).all()
    with pytest.raises(T.TcabError) as e:       # the value per row of the innermost-axis kernels is not a value per cell
        T.chain_reduce([xd, torch.zeros((nb, nk, 1), device=cuda)], "p0 * p1", axis=1)
    assert e.value.status == T._lib.ERR_SHAPE


def test_bound_chain_reduce_is_the_same_call(cuda):
    """Descriptors built once, launched many times: the same results and one launch per call."""
    rng = np.random.default_rng(11)
    x = to_dev(rng.uniform(-1, 1, (300, 1001)).astype(np.float32), cuda)
    z = to_dev(rng.uniform(0, 1, (300, 1001)).astype(np.float32), cuda)
    want = T.chain_reduce([x, z], "p0 * p1 + c0", captures=(0.5,), init=1.0, post_expr="p0 * 2.0f")
    call = T.BoundChainReduce([x, z], "p0 * p1 + c0", captures=(0.5,), init=1.0, post_expr="p0 * 2.0f")
    n0 = T.launch_count()
    for _ in range(3):
        got = call()
    assert T.launch_count() - n0 == 3
    assert torch.equal(got, want)
    x.mul_(2.0)                                     # the operands are read at every call
    assert torch.equal(call(), T.chain_reduce([x, z], "p0 * p1 + c0", captures=(0.5,), init=1.0, post_expr="p0 * 2.0f"))
    mid = T.BoundChainReduce([x.view(3, 100, 1001)], "p0", combine_expr="fmaxf(p0, p1)", init=-10.0, axis=1)
    assert torch.equal(mid(), x.view(3, 100, 1001).max(1).values)
    with pytest.raises(ValueError):
        T.BoundChainReduce([x, z.cpu()], "p0 * p1")


@pytest.mark.parametrize("shape,axis", [((3000, 1024), 1), ((700, 8192), 1), ((5, 400000), 1), ((2000, 520), 1), ((1500, 1032), 1),
                                        ((40, 300, 512), 1), ((3, 5000, 256), 1), ((200, 64, 1024), 1), ((9, 100, 264), 1)])
def test_chains_whose_operands_are_all_bf16(cuda, shape, axis):
    """Every operand bf16: rows of whole 16-byte vectors are read as vectors of eight (innermost axis beyond 512 columns,
    middle axis from 256 columns), everything else as before; sums against fp64, max bit-exact."""
    from oracle import binding as O
    rng = np.random.default_rng(sum(shape))
    xb = O.f32_to_bf16(rng.uniform(-1, 1, shape).astype(np.float32))
    zb = O.f32_to_bf16(rng.uniform(0, 1, shape).astype(np.float32))
    x64, z64 = O.bf16_to_f32(xb).astype(np.float64), O.bf16_to_f32(zb).astype(np.float64)
    xd, zd = to_dev(xb, cuda), to_dev(zb, cuda)
    got = T.chain_reduce([xd], "f32(p0)", axis=axis).cpu().numpy()
    assert (np.abs(got - x64.sum(axis)) <= 1e-5 * np.abs(x64).sum(axis) + 1e-30).all()
    got = T.chain_reduce([xd, zd], "f32(p0) * f32(p1) + c0", captures=(0.25,), init=1.0, axis=axis, post_expr="p0 * 0.5f").cpu().numpy()
    want = ((x64 * z64 + 0.25).sum(axis) + 1.0) * 0.5
    assert (np.abs(got - want) <= 1e-5 * (np.abs(x64 * z64) + 0.25).sum(axis) + 1e-5).all()
    got = T.chain_reduce([xd], "f32(p0)", combine_expr="fmaxf(p0, p1)", init=-2.0, axis=axis).cpu().numpy()
    assert np.array_equal(got, O.bf16_to_f32(xb).max(axis))


def test_bf16_map_results_round_like_the_oracle(cuda):
    """The map kernels convert two results at a time with the conversion instruction: round to nearest even on every
    value, infinities kept, and a NaN keeps its sign and payload as the oracle's conversion does."""
    from oracle import binding as O
    rng = np.random.default_rng(5)
    x = rng.normal(0, 1, (257, 1000)).astype(np.float32)
    x[0, :8] = [np.inf, -np.inf, np.nan, -np.nan, 3.3895314e38, -3.3895314e38, 1e-40, -1e-45]   # the last four: overflow to inf, denormals
    x.view(np.uint32)[1, :4] = [0x7FC12345, 0xFF812345, 0x7F800001, 0x3F808000]               # NaN payloads; a tie
    x.view(np.uint32)[2, :1000] = (0x3F800000 + rng.integers(0, 1 << 17, 1000)).astype(np.uint32)  # values around the ties
    got = T.map([to_dev(x, cuda)], "bf16(p0)", out_dtype=torch.bfloat16)
    bits = got.view(torch.int16).cpu().numpy().view(np.uint16)
    assert np.array_equal(bits, O.f32_to_bf16(x))
