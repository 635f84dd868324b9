"""Parity of the CUDA kernels (through the C ABI) with the CPU oracle on a B200.

Tolerances, as stated for this path:
  * integer / index outputs (argmax) and max: bit-exact;
  * fp32 reductions: |gpu - oracle| <= 1e-5 relative, with the denominators
    written at each test (normwise max|ref|, and per element sum|x_i| where the
    sum cancels). The oracle folds sequentially in fp32, as the reference's
    loops do, and for long rows that fold is itself further than 1e-5 from the
    exact value (measured: 1.5e-5 at 4096 terms, 1.8e-5 at 70001) while the
    kernel's tree is within 3e-6. Where that matters the bound is
        |gpu - oracle| <= 1e-5*|oracle| + |oracle - fp64|   and   |gpu - fp64| <= 1e-5*|fp64|,
    fp64 being the same formula evaluated in double precision on the same inputs;
  * softmax / layer-norm outputs (a map after reductions): the same bound for
    fp32; for bf16 outputs one bf16 ulp of the value plus the fp32 error of the
    terms that cancel in x_hat*gamma + beta.
Every output buffer is prefilled with a canary and padded with guard bands, the
reference's own way of proving that every element was written and nothing else
(internal/e2e/harness.go:158-181, testing/runners/common.cuh).
"""
import json
import os

import numpy as np
import pytest
import torch

import tcacomp_b200 as T
from guards import guarded_input

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))
GOLDEN = json.load(open(os.path.join(HERE, "golden", "suite_golden.json")))
CANARY = -12345.0
GUARD = 64


def guarded(shape, dtype, dev):
    """An output view with CANARY-filled guard bands on both sides of it."""
    n = int(np.prod(shape))
    buf = torch.full((n + 2 * GUARD,), CANARY, dtype=torch.float32, device=dev).to(dtype)
    return buf, buf[GUARD:GUARD + n].view(*shape)


def check_guards(buf, dtype):
    b = buf.float().cpu().numpy()
    want = torch.tensor(CANARY).to(dtype).float().item()
    assert (b[:GUARD] == want).all() and (b[-GUARD:] == want).all(), "kernel wrote outside its output"


def dev_f32(a, dev):
    return guarded_input(a, dev)       # NaN bands around every operand: a read outside it cannot pass by luck


def dev_bf16(bits, dev):
    return guarded_input(bits, dev)    # uint16 bit patterns -> a bf16 tensor inside NaN bands


def host_bits(t):
    return t.view(torch.int16).cpu().numpy().view(np.uint16)


# ----------------------------------------------------------------------------
# fused map + innermost-axis reduce
# ----------------------------------------------------------------------------
@pytest.mark.parametrize("rows,cols", [(4096, 1024), (1, 1), (3, 5), (37, 130), (64, 32), (129, 264),
                                       (5, 9000), (2, 70001), (1000, 4)])
def test_map_rowsum(oracle, cuda, rows, cols, parity_counts):
    # (4096, 1024) is the benchmark configuration; every output element of it is compared with the oracle
    rng = np.random.default_rng(rows * 131 + cols)
    x = rng.uniform(-1, 1, (rows, cols)).astype(np.float32)
    want = oracle.map_rowsum_affine_sq(x)
    buf, out = guarded((rows,), torch.float32, cuda)
    T.chain_reduce([dev_f32(x, cuda)], "(0.5f*p0 + 0.25f) * (0.5f*p0 + 0.25f)", out=out)
    got = out.cpu().numpy()
    check_guards(buf, torch.float32)
    assert (got != CANARY).all()
    from oracle import checks
    rep = checks.rowsum_report(got, x)
    if (rows, cols) == (4096, 1024):
        parity_counts["C1 map+rowsum f32 [4096,1024]"] = rep.as_dict()
    assert rep.ok, rep


def test_map_rowsum_unaligned_and_captures(oracle, cuda):
    rng = np.random.default_rng(1)
    x = rng.uniform(-1, 1, (33, 1024)).astype(np.float32)
    base = torch.zeros(33 * 1024 + 1, device=cuda)
    xd = base[1:].view(33, 1024)  # 4-byte aligned only: the scalar path
    xd.copy_(dev_f32(x, cuda))
    got = T.chain_reduce([xd], "(c0*p0 + c1) * (c0*p0 + c1)", captures=(0.5, 0.25)).cpu().numpy()
    want = oracle.map_rowsum_affine_sq(x)
    assert np.abs(got - want).max() <= 1e-5 * np.abs(want).max()


@pytest.mark.parametrize("op,expr,init", [("sum", "(p0 + p1)", 0.0), ("max", "fmaxf(p0, p1)", -np.inf),
                                          ("min", "fminf(p0, p1)", np.inf), ("sum", "(p0 + p1)", 2.5)])
def test_row_reduce_ops_and_init(oracle, cuda, op, expr, init):
    rng = np.random.default_rng(2)
    for rows, cols in [(17, 300), (4, 4), (2, 5000)]:
        x = rng.normal(0, 3, (rows, cols)).astype(np.float32)
        want = oracle.row_reduce(x, op, init)
        got = T.chain_reduce([dev_f32(x, cuda)], "p0", combine_expr=expr, init=float(init)).cpu().numpy()
        if op == "sum":
            assert (np.abs(got - want) <= 1e-5 * np.abs(x).sum(1)).all()
        else:
            assert np.array_equal(got, want)  # max/min are order-independent: bit-exact
    # empty reduction returns init (design/tca.md:299)
    e = torch.zeros((6, 0), device=cuda)
    got = T.chain_reduce([e], "p0", combine_expr=expr, init=float(init)).cpu().numpy()
    assert np.array_equal(got, np.full(6, init, np.float32))


def test_thread_per_row_is_bit_exact(oracle, cuda):
    # rows of <= 32 elements are folded by one thread in ascending order: the reference's
    # SeqReducer order (runtime/tca/reducer.h:45-51), so even sums match bit for bit
    rng = np.random.default_rng(4)
    x = rng.uniform(-1, 1, (513, 32)).astype(np.float32)
    got = T.chain_reduce([dev_f32(x, cuda)], "p0").cpu().numpy()
    assert np.array_equal(got, oracle.row_reduce(x, "sum", 0.0))


# ----------------------------------------------------------------------------
# the reference's suite kernels that are reductions of identically shaped operands
# ----------------------------------------------------------------------------
SUITE_CHAINS = {
    # name: (map, post, axis, captures)
    "row_sum": ("(p0 * p1)", None, 1, ()),
    "softmax": ("(expf(p0) * p1)", None, 1, ()),
    "transpose": ("(p0 * p1)", None, 2, ()),
    "scale_copy": ("((c0 * p0) + c1) * p1", None, 2, (1.25, -0.125)),
    "axpy3": ("c0 * p0 + c1 * p1", "p0 + c2 * tanhf(p0)", 2, (2.0, 0.5, 0.75)),
    "layernorm": ("(p0 * p0) * p1", "p0 * rsqrtf(p0 * c0 + c1)", 2, (1.0 / 64.0, 1e-5)),
}
SUITE_TOL = {"row_sum": 2e-3, "softmax": 2e-3, "transpose": 1e-5, "scale_copy": 1e-5, "axpy3": 1e-5,
             "layernorm": 1e-5}  # testing/suite.toml tolerances (max abs diff)


@pytest.mark.parametrize("name", sorted(SUITE_CHAINS))
def test_reference_suite_kernels(oracle, cuda, name):
    mp, post, axis, caps = SUITE_CHAINS[name]
    x, z = oracle.suite_inputs(name)
    want = oracle.suite(name)
    g = GOLDEN[name]
    assert abs(want.astype(np.float64).sum() - g["checksum"]) <= 1e-6 * abs(g["checksum"])
    buf, out = guarded(want.shape, torch.float32, cuda)
    T.chain_reduce([dev_f32(x, cuda), dev_f32(z, cuda)], mp, post_expr=post, captures=caps, axis=axis, out=out)
    got = out.cpu().numpy()
    check_guards(buf, torch.float32)
    assert (got == CANARY).sum() == 0  # the runner's CANARY line
    assert np.abs(got.astype(np.float64) - want).max() <= SUITE_TOL[name]  # the runner's MAXDIFF line
    assert abs(got.astype(np.float64).sum() - g["checksum"]) <= 1e-5 * abs(g["checksum"])


def test_e2e_row_sum_fixture(oracle, cuda):
    # internal/e2e/e2e_test.go:15-21,300-330: 1024 x 512 row sums of elem(i), tolerance 2e-3 absolute
    x = oracle.elem_fill(1024 * 512).reshape(1024, 512)
    got = T.chain_reduce([dev_f32(x, cuda)], "p0").cpu().numpy()
    g = GOLDEN["e2e_row_sum_1024x512"]
    assert np.abs(got - oracle.row_reduce(x, "sum", 0.0)).max() <= 2e-3
    assert abs(got.astype(np.float64).sum() - g["checksum"]) <= 1e-5 * g["checksum"]


# ----------------------------------------------------------------------------
# row softmax
# ----------------------------------------------------------------------------
def assert_softmax_close(got, want, x):
    from oracle import checks
    assert checks.softmax_close(got, x, want)


@pytest.mark.parametrize("rows,cols", [(64, 4096), (1, 1), (3, 7), (33, 517), (130, 32), (7, 1000), (5, 12288),
                                       (3, 40000), (2, 140004), (2, 140001),
                                       # thread-block clusters of 2, 4, 8 CTAs (vector and scalar paths) and
                                       # the first size past them
                                       (2, 32772), (5, 60000), (3, 50001), (2, 262144), (1, 262148),
                                       # rows that are not a multiple of four columns: 16-byte vectors with
                                       # element-wise row ends, every head offset 0..3, one CTA and clusters
                                       (9, 17), (301, 4097), (40, 8191), (7, 8194), (6, 12289), (5, 50257), (4, 65539),
                                       (5, 131071)])
def test_softmax_rows(oracle, cuda, rows, cols):
    rng = np.random.default_rng(rows * 7 + cols)
    x = (4 * rng.normal(0, 1, (rows, cols))).astype(np.float32)
    want = oracle.softmax_rows(x)
    buf, out = guarded((rows, cols), torch.float32, cuda)
    T.softmax_rows(dev_f32(x, cuda), out=out)
    got = out.cpu().numpy()
    check_guards(buf, torch.float32)
    assert_softmax_close(got, want, x)
    assert np.abs(got.astype(np.float64).sum(1) - 1.0).max() <= 1e-5


@pytest.mark.parametrize("rows,cols,cs,shape", [(80, 24576, 0, 0), (75, 49152, 0, 0), (74, 98308, 0, 0),   # the library's own choice
                                                 (76, 50257, 0, 0), (77, 32003, 0, 0), (33, 131076, 0, 0), (2, 300004, 0, 0), (5, 4099, 2, 1), (6, 1001, 4, 1),
                                                 (3, 70001, 8, 3), (4, 14, 2, 1), (9, 9, 8, 1),
                                                 (3, 4096, 2, 1), (2, 12292, 3, 1), (5, 1028, 8, 1), (2, 65536, 4, 2),
                                                 (3, 40000, 5, 3), (1, 300000, 8, 4), (2, 262148, 8, 5), (1, 1048576, 8, 5),
                                                 (7, 20, 8, 1)])
def test_softmax_streaming_clusters(oracle, cuda, rows, cols, cs, shape):
    # long rows: a cluster streams the row twice (the second time from L2) with an online max / sum in the first
    # pass; forced shapes include clusters with CTAs that get no element at all
    rng = np.random.default_rng(rows + cols + cs)
    x = (4 * rng.normal(0, 1, (rows, cols))).astype(np.float32)
    x[0, :: max(2, cols // 7)] = -np.inf            # -inf entries add nothing
    x[rows - 1, cols // 3:] -= 40.0                 # the maximum sits early in the row: later segments rescale
    buf, out = guarded((rows, cols), torch.float32, cuda)
    n0 = T.launch_count()
    try:
        if cs:
            T.tune("softmax", 0, cs, shape, 7)
        T.softmax_rows(dev_f32(x, cuda), out=out)
    finally:
        T.tune("softmax")
    assert T.launch_count() - n0 == 1
    got = out.cpu().numpy()
    check_guards(buf, torch.float32)
    assert_softmax_close(got, oracle.softmax_rows(x), x)
    assert np.abs(got.astype(np.float64).sum(1) - 1.0).max() <= 1e-5
    # an all -inf row is NaN, like the plain formula; one finite entry takes everything
    xx = np.full((2, cols), -np.inf, np.float32)
    xx[1, cols // 2] = 5.0
    try:
        T.tune("softmax", 0, cs or 2, shape or 1, 7)
        g = T.softmax_rows(dev_f32(xx, cuda)).cpu().numpy()
    finally:
        T.tune("softmax")
    assert np.isnan(g[0]).all() and g[1, cols // 2] == 1.0 and g[1].sum() == 1.0


def test_softmax_unaligned_view(oracle, cuda):
    rng = np.random.default_rng(12)
    x = (4 * rng.normal(0, 1, (9, 256))).astype(np.float32)
    base = torch.zeros(9 * 256 + 3, device=cuda)
    xd = base[3:].view(9, 256)
    xd.copy_(dev_f32(x, cuda))
    got = T.softmax_rows(xd).cpu().numpy()
    assert_softmax_close(got, oracle.softmax_rows(x), x)


def test_softmax_extremes(oracle, cuda):
    x = np.array([[1e4, -1e4, 0, 88.0], [-np.inf, 0.0, 1.0, -np.inf], [3.0, 3.0, 3.0, 3.0]], np.float32)
    got = T.softmax_rows(dev_f32(x, cuda)).cpu().numpy()
    want = oracle.softmax_rows(x)
    assert np.allclose(got, want, rtol=1e-5, atol=0)
    for cols in (4, 140004):  # the register-resident kernel and the online one
        xx = np.full((2, cols), -np.inf, np.float32)
        xx[1, cols // 2] = 5.0
        g = T.softmax_rows(dev_f32(xx, cuda)).cpu().numpy()
        assert np.isnan(g[0]).all() and g[1, cols // 2] == 1.0 and g[1].sum() == 1.0


def test_softmax_full_size_every_element(oracle, cuda, parity_counts):
    # the benchmark configuration: fp32 [16384, 4096] ~ 4*N(0,1); every output element against the oracle
    # (testing/runners/softmax.cu:49-61 is the loop the oracle restates)
    gen = torch.Generator(device=cuda).manual_seed(2024)
    x = 4 * torch.randn((16384, 4096), generator=gen, device=cuda)
    y = T.softmax_rows(x)
    s = y.double().sum(1)
    assert (s - 1).abs().max().item() <= 1e-5
    # the largest input of a row receives the largest output
    assert (y >= 0).all() and torch.equal(y.gather(1, x.argmax(1, keepdim=True)).squeeze(1), y.amax(1))
    from oracle import checks
    rep = checks.softmax_report_fast(y.cpu().numpy(), x.cpu().numpy())
    parity_counts["C2 softmax f32 [16384,4096]"] = rep.as_dict()
    assert rep.checked == 16384 * 4096 and rep.ok, rep


# ----------------------------------------------------------------------------
# layer-norm
# ----------------------------------------------------------------------------
def assert_layernorm_bf16_close(oracle, got_bits, want_bits, x_bits, g_bits, b_bits, eps=1e-5):
    from oracle import checks
    assert checks.layernorm_bf16_close(got_bits, x_bits, g_bits, b_bits, eps, want_bits)


@pytest.mark.parametrize("rows,cols", [(64, 8192), (1, 1), (3, 7), (17, 264), (130, 64), (9, 1000), (4, 16384),
                                       (3, 70000), (2, 300008)])
def test_layernorm_rows_bf16(oracle, cuda, rows, cols):
    rng = np.random.default_rng(rows * 3 + cols)
    x = oracle.f32_to_bf16(rng.normal(0, 1, (rows, cols)).astype(np.float32))
    g = oracle.f32_to_bf16(rng.normal(1, 0.1, cols).astype(np.float32))
    b = oracle.f32_to_bf16(rng.normal(0, 0.1, cols).astype(np.float32))
    want = oracle.layernorm_rows_bf16(x, g, b, 1e-5)
    buf, out = guarded((rows, cols), torch.bfloat16, cuda)
    T.layernorm_rows(dev_bf16(x, cuda), dev_bf16(g, cuda), dev_bf16(b, cuda), 1e-5, out=out)
    got = host_bits(out)
    check_guards(buf, torch.bfloat16)
    assert_layernorm_bf16_close(oracle, got, want, x, g, b)


@pytest.mark.parametrize("rows,cols", [(33, 1024), (5, 77), (3, 20000), (2, 131072), (2, 50001)])
def test_layernorm_rows_f32(oracle, cuda, rows, cols):
    rng = np.random.default_rng(cols)
    x = rng.normal(0, 1, (rows, cols)).astype(np.float32)
    g = rng.normal(1, 0.1, cols).astype(np.float32)
    b = rng.normal(0, 0.1, cols).astype(np.float32)
    want = oracle.layernorm_rows_f32(x, g, b, 1e-5)
    got = T.layernorm_rows(dev_f32(x, cuda), dev_f32(g, cuda), dev_f32(b, cuda), 1e-5).cpu().numpy()
    x64 = x.astype(np.float64)
    y64 = (x64 - x64.mean(1, keepdims=True)) / np.sqrt(x64.var(1, keepdims=True) + 1e-5) * g + b
    scale = np.abs(y64).max()
    assert np.abs(got - y64).max() <= 1e-5 * scale
    # against the oracle, charged with its own sequential-fold distance from the fp64 value
    assert np.abs(got - want).max() <= 1e-5 * scale + np.abs(want - y64).max()


@pytest.mark.parametrize("rows,cols", [(19, 33), (17, 127), (21, 130), (11, 1001), (9, 4097), (10, 8191), (9, 10001),
                                       (5, 20001), (9, 32767), (3, 32769)])
@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_layernorm_rows_not_whole_vectors(oracle, cuda, rows, cols, dtype):
    # rows that start at every offset inside a 16-byte vector: edge elements, shifted gamma / beta, guarded output
    rng = np.random.default_rng(rows * 7 + cols)
    x = rng.normal(0.3, 1, (rows, cols)).astype(np.float32)
    g = rng.normal(1, 0.1, cols).astype(np.float32)
    b = rng.normal(0, 0.1, cols).astype(np.float32)
    if dtype == "f32":
        want = oracle.layernorm_rows_f32(x, g, b, 1e-5)
        buf, out = guarded((rows, cols), torch.float32, cuda)
        T.layernorm_rows(dev_f32(x, cuda), dev_f32(g, cuda), dev_f32(b, cuda), 1e-5, out=out)
        got = out.cpu().numpy()
        check_guards(buf, torch.float32)
        x64 = x.astype(np.float64)
        y64 = (x64 - x64.mean(1, keepdims=True)) / np.sqrt(x64.var(1, keepdims=True) + 1e-5) * g + b
        scale = np.abs(y64).max()
        assert np.abs(got - y64).max() <= 1e-5 * scale
        assert np.abs(got - want).max() <= 1e-5 * scale + np.abs(want - y64).max()
    else:
        xb, gb, bb = oracle.f32_to_bf16(x), oracle.f32_to_bf16(g), oracle.f32_to_bf16(b)
        buf, out = guarded((rows, cols), torch.bfloat16, cuda)
        T.layernorm_rows(dev_bf16(xb, cuda), dev_bf16(gb, cuda), dev_bf16(bb, cuda), 1e-5, out=out)
        got = host_bits(out)
        check_guards(buf, torch.bfloat16)
        assert_layernorm_bf16_close(oracle, got, oracle.layernorm_rows_bf16(xb, gb, bb, 1e-5), xb, gb, bb)
        # the 2-byte path computes the same statistics; the two may differ by a rounding on few elements
        try:
            T.tune("layernorm", 0, 0, 0, 6)
            plain = host_bits(T.layernorm_rows(dev_bf16(xb, cuda), dev_bf16(gb, cuda), dev_bf16(bb, cuda), 1e-5))
        finally:
            T.tune("layernorm")
        assert (plain != got).mean() <= 0.02


@pytest.mark.parametrize("cols", [32776, 100000, 20001, 262144])
def test_layernorm_cluster_kernel_forced(oracle, cuda, cols):
    # the thread-block-cluster kernel is a heuristic choice; force it so that every cluster size is checked
    rng = np.random.default_rng(cols)
    x = oracle.f32_to_bf16(rng.normal(0, 1, (3, cols)).astype(np.float32))
    g = oracle.f32_to_bf16(rng.normal(1, 0.1, cols).astype(np.float32))
    b = oracle.f32_to_bf16(rng.normal(0, 0.1, cols).astype(np.float32))
    try:
        T.tune("layernorm", 0, 0, 0, 3)
        got = host_bits(T.layernorm_rows(dev_bf16(x, cuda), dev_bf16(g, cuda), dev_bf16(b, cuda)))
    finally:
        T.tune("layernorm")
    assert_layernorm_bf16_close(oracle, got, oracle.layernorm_rows_bf16(x, g, b, 1e-5), x, g, b)


@pytest.mark.parametrize("dtype,rows,cols,cs,shape", [("f32", 80, 24576, 0, 0), ("f32", 75, 45056, 0, 0), ("bf16", 74, 131072, 0, 0),
                                                       ("f32", 3, 65540, 0, 0), ("bf16", 2, 262152, 0, 0),
                                                       ("f32", 3, 4096, 2, 1), ("f32", 2, 12292, 3, 4), ("f32", 5, 1028, 8, 1),
                                                       ("f32", 2, 65536, 4, 2), ("f32", 1, 300000, 8, 5), ("f32", 7, 20, 8, 1),
                                                       ("bf16", 3, 8192, 2, 1), ("bf16", 2, 65544, 5, 3), ("bf16", 1, 300008, 8, 5),
                                                       ("bf16", 6, 40, 8, 4)])
def test_layernorm_streaming_clusters(oracle, cuda, dtype, rows, cols, cs, shape):
    # long rows: a cluster streams the row (statistics from shifted sums in one pass; a centred pass when the shift
    # turns out far from the mean), then once more from L2 to normalise. Row 0 has a mean far from its first
    # element (the centred pass runs), the other rows do not; forced shapes include CTAs without any element.
    rng = np.random.default_rng(rows + cols + cs)
    x = rng.normal(0.2, 1, (rows, cols)).astype(np.float32)
    x[0] += 7.0
    x[0, 0] = 4.0          # the shift K: three standard deviations below the row's mean
    g = rng.normal(1, 0.1, cols).astype(np.float32)
    b = rng.normal(0, 0.1, cols).astype(np.float32)
    n0 = T.launch_count()
    try:
        if cs:
            T.tune("layernorm", 0, cs, shape, 7)
        if dtype == "f32":
            buf, out = guarded((rows, cols), torch.float32, cuda)
            T.layernorm_rows(dev_f32(x, cuda), dev_f32(g, cuda), dev_f32(b, cuda), 1e-5, out=out)
        else:
            xb, gb, bb = oracle.f32_to_bf16(x), oracle.f32_to_bf16(g), oracle.f32_to_bf16(b)
            buf, out = guarded((rows, cols), torch.bfloat16, cuda)
            T.layernorm_rows(dev_bf16(xb, cuda), dev_bf16(gb, cuda), dev_bf16(bb, cuda), 1e-5, out=out)
    finally:
        T.tune("layernorm")
    assert T.launch_count() - n0 == 1
    if dtype == "f32":
        got = out.cpu().numpy()
        check_guards(buf, torch.float32)
        want = oracle.layernorm_rows_f32(x, g, b, 1e-5)
        x64 = x.astype(np.float64)
        y64 = (x64 - x64.mean(1, keepdims=True)) / np.sqrt(x64.var(1, keepdims=True) + 1e-5) * g + b
        scale = np.abs(y64).max()
        assert np.abs(got - y64).max() <= 1e-5 * scale
        assert np.abs(got - want).max() <= 1e-5 * scale + np.abs(want - y64).max()
    else:
        got = host_bits(out)
        check_guards(buf, torch.bfloat16)
        assert_layernorm_bf16_close(oracle, got, oracle.layernorm_rows_bf16(xb, gb, bb, 1e-5), xb, gb, bb)


@pytest.mark.parametrize("cache", [0, 1])
def test_layernorm_variants_agree(oracle, cuda, cache):
    rng = np.random.default_rng(77)
    x = oracle.f32_to_bf16(rng.normal(0, 1, (300, 8192)).astype(np.float32))
    g = oracle.f32_to_bf16(rng.normal(1, 0.1, 8192).astype(np.float32))
    b = oracle.f32_to_bf16(rng.normal(0, 0.1, 8192).astype(np.float32))
    try:
        T.tune("layernorm", 0, 0, 0, cache)
        got = host_bits(T.layernorm_rows(dev_bf16(x, cuda), dev_bf16(g, cuda), dev_bf16(b, cuda)))
    finally:
        T.tune("layernorm")
    assert_layernorm_bf16_close(oracle, got, oracle.layernorm_rows_bf16(x, g, b, 1e-5), x, g, b)


def test_layernorm_full_size_every_element(oracle, cuda, parity_counts):
    # the benchmark configuration: bf16 [65536, 8192]; every output element against the oracle
    # (testing/runners/layernorm.cu:47-58 is the loop the oracle restates), in slabs of rows
    gen = torch.Generator(device=cuda).manual_seed(7)
    x = torch.randn((65536, 8192), generator=gen, device=cuda, dtype=torch.float32).to(torch.bfloat16)
    g = (1 + 0.1 * torch.randn(8192, generator=gen, device=cuda)).to(torch.bfloat16)
    b = (0.1 * torch.randn(8192, generator=gen, device=cuda)).to(torch.bfloat16)
    y = T.layernorm_rows(x, g, b, 1e-5)
    from oracle import checks
    rep = checks.layernorm_bf16_report_fast(host_bits(y), host_bits(x), host_bits(g), host_bits(b))
    parity_counts["C3 layer-norm bf16 [65536,8192]"] = rep.as_dict()
    assert rep.checked == 65536 * 8192 and rep.ok, rep
    # with gamma = 1, beta = 0 every output row has mean ~0 and variance ~1
    one, zero = torch.ones_like(g), torch.zeros_like(b)
    y1 = T.layernorm_rows(x[:4096], one, zero, 1e-5).float()
    assert y1.mean(1).abs().max().item() < 5e-3 and (y1.var(1, unbiased=False) - 1).abs().max().item() < 2e-2


# ----------------------------------------------------------------------------
# outer-axis reduce: sum / max / argmax
# ----------------------------------------------------------------------------
@pytest.mark.parametrize("nb,nk,nc", [(4, 1024, 1024), (1, 1, 1), (3, 37, 50), (2, 5, 129), (5, 300, 4), (2, 1000, 260),
                                      (1, 9, 2000)])
def test_reduce_outer(oracle, cuda, nb, nk, nc):
    rng = np.random.default_rng(nb * 1000 + nk + nc)
    t = rng.uniform(-100, 100, (nb, nk, nc)).astype(np.float32)
    s, m, a = oracle.reduce_outer(t)
    bs, os_ = guarded((nb, nc), torch.float32, cuda)
    bm, om = guarded((nb, nc), torch.float32, cuda)
    oa_i = torch.full((nb, nc), -7, dtype=torch.int32, device=cuda)
    T.reduce_outer(dev_f32(t, cuda), out={"sum": os_, "max": om, "argmax": oa_i})
    check_guards(bs, torch.float32)
    check_guards(bm, torch.float32)
    assert np.array_equal(om.cpu().numpy(), m)            # bit-exact
    assert np.array_equal(oa_i.cpu().numpy(), a)          # bit-exact, lowest index on ties
    got = os_.cpu().numpy()
    _, sabs = oracle.reduce_outer_sum_f64(t)
    assert (np.abs(got - s) <= 1e-5 * sabs).all()          # per element against sum|x_i|
    assert np.abs(got - s).max() <= 1e-5 * max(np.abs(s).max(), 1.0)  # normwise


def test_reduce_outer_ties_and_subsets(oracle, cuda):
    rng = np.random.default_rng(99)
    t = rng.integers(-3, 4, (6, 200, 132)).astype(np.float32)  # many equal maxima
    t[0, :, 0] = 2.0
    t[1, 150:, 5] = 3.0
    s, m, a = oracle.reduce_outer(t)
    td = dev_f32(t, cuda)
    r = T.reduce_outer(td)
    assert np.array_equal(r["argmax"].cpu().numpy(), a) and np.array_equal(r["max"].cpu().numpy(), m)
    assert np.array_equal(r["sum"].cpu().numpy(), s)  # small integers: every order gives the exact sum
    only = T.reduce_outer(td, want=("argmax",))
    assert set(only) == {"argmax"} and np.array_equal(only["argmax"].cpu().numpy(), a)
    # NaN never wins a strict '>' comparison; an all-NaN column keeps (-inf, 0)
    t2 = t.copy()
    t2[2, 3, 7] = np.nan
    t2[3, :, 9] = np.nan
    s2, m2, a2 = oracle.reduce_outer(t2)
    r2 = T.reduce_outer(dev_f32(t2, cuda), want=("max", "argmax"))
    assert np.array_equal(r2["argmax"].cpu().numpy(), a2)
    assert np.array_equal(r2["max"].cpu().numpy(), m2, equal_nan=True)
    # empty reduction: the inits (design/tca.md:299)
    e = T.reduce_outer(torch.zeros((2, 0, 8), device=cuda))
    assert (e["sum"] == 0).all() and torch.isneginf(e["max"]).all() and (e["argmax"] == 0).all()


@pytest.mark.parametrize("cv,kw", [(1, 8), (2, 8), (1, 16), (2, 16), (1, 4), (2, 4)])
def test_reduce_outer_all_launch_shapes(oracle, cuda, cv, kw):
    rng = np.random.default_rng(cv * 10 + kw)
    t = rng.uniform(-100, 100, (3, 77, 392)).astype(np.float32)
    s, m, a = oracle.reduce_outer(t)
    try:
        T.tune("reduce_outer", cv, kw)
        r = T.reduce_outer(dev_f32(t, cuda))
    finally:
        T.tune("reduce_outer")
    assert np.array_equal(r["argmax"].cpu().numpy(), a) and np.array_equal(r["max"].cpu().numpy(), m)
    assert np.abs(r["sum"].cpu().numpy() - s).max() <= 1e-5 * np.abs(t).sum(1).max()


def test_reduce_outer_full_size_every_element(oracle, cuda, parity_counts):
    # the benchmark configuration: fp32 [256, 1024, 1024] ~ U(-100, 100); every output against the oracle
    gen = torch.Generator(device=cuda).manual_seed(5)
    t = torch.rand((256, 1024, 1024), generator=gen, device=cuda) * 200 - 100
    r = T.reduce_outer(t)
    # argmax indexes the max: gather(t, argmax) == max, bit for bit; and max >= every element
    picked = torch.gather(t, 1, r["argmax"].long().unsqueeze(1)).squeeze(1)
    assert torch.equal(picked, r["max"])
    assert torch.equal(r["max"], t.amax(1))
    # linearity of the sum: sum(2*t) == 2*sum(t) exactly (scaling by 2 is exact in fp32)
    r2 = T.reduce_outer(t * 2, want=("sum",))
    assert torch.equal(r2["sum"], r["sum"] * 2)
    from oracle import checks
    rep = checks.Report()
    for lo in range(0, 256, 16):   # slabs of 16 batches: 64 MiB of input on the host at a time
        sl = t[lo:lo + 16].cpu().numpy()
        s, m, a = oracle.reduce_outer(sl)
        assert np.array_equal(r["argmax"][lo:lo + 16].cpu().numpy(), a), lo     # bit-exact, lowest index on ties
        assert np.array_equal(r["max"][lo:lo + 16].cpu().numpy(), m), lo       # bit-exact
        rep.merge(checks.outer_sum_report(r["sum"][lo:lo + 16].cpu().numpy(), s, sl))
    parity_counts["C4 outer sum f32 [256,1024,1024] (max and argmax bit-exact on all)"] = rep.as_dict()
    assert rep.checked == 256 * 1024 and rep.ok, rep


@pytest.mark.parametrize("nb,nk,nc,forced", [(1, 100000, 64, 0), (2, 5000, 100, 0), (1, 70001, 33, 0), (3, 1000, 132, 7),
                                              (1, 300, 8, 300), (2, 4097, 260, 5)])
def test_reduce_outer_k_split_over_ctas(oracle, cuda, nb, nk, nc, forced):
    # few columns, long k: the k axis is split over CTAs and the partial states are folded by a second kernel
    rng = np.random.default_rng(nk + nc)
    t = rng.integers(-50, 51, (nb, nk, nc)).astype(np.float32)  # integers: many equal maxima, exact sums
    t[0, nk // 2:, 1] = 50.0                                   # a tie that spans several k ranges
    t[0, :, 2] = -np.inf
    t[0, 5, 3] = np.inf
    t[nb - 1, 7, 4] = np.nan
    s, m, a = oracle.reduce_outer(t)
    n0 = T.launch_count()
    try:
        T.tune("reduce_outer", 0, 0, 0, forced)
        r = T.reduce_outer(dev_f32(t, cuda))
    finally:
        T.tune("reduce_outer")
    assert T.launch_count() - n0 == 2, "expected the split kernel plus the finishing kernel"
    assert np.array_equal(r["argmax"].cpu().numpy(), a)
    assert np.array_equal(r["max"].cpu().numpy(), m, equal_nan=True)
    got = r["sum"].cpu().numpy()
    finite = np.isfinite(s)
    assert np.array_equal(got[finite], s[finite])
    assert np.array_equal(np.isnan(got), np.isnan(s)) and np.array_equal(np.isinf(got), np.isinf(s))
    only = T.reduce_outer(dev_f32(t, cuda), want=("max",))
    assert np.array_equal(only["max"].cpu().numpy(), m, equal_nan=True)


@pytest.mark.parametrize("rows,cols", [(3, 4096), (151, 12288), (300, 8200), (149, 45056), (5, 16), (450, 4100),
                                       (310, 18000), (150, 36000)])
def test_rows_in_shared_memory(oracle, cuda, rows, cols):
    # the shared-memory row kernels (bulk asynchronous copies into a ring of slots, three passes), forced through the
    # tuning hook: one slot and many, a ragged last slot, fewer rows than SMs and several rows per CTA
    rng = np.random.default_rng(rows + cols)
    x = (4 * rng.normal(0, 1, (rows, cols))).astype(np.float32)
    x[0, :7] = -np.inf
    buf, out = guarded((rows, cols), torch.float32, cuda)
    try:
        T.tune("softmax", 0, 0, 0, 3)
        n0 = T.launch_count()
        T.softmax_rows(dev_f32(x, cuda), out=out)
        assert T.launch_count() - n0 == 1
    finally:
        T.tune("softmax")
    check_guards(buf, torch.float32)
    from oracle import checks
    assert checks.softmax_close(out.cpu().numpy(), x)
    g32 = rng.normal(1, 0.1, cols).astype(np.float32)
    b32 = rng.normal(0, 0.1, cols).astype(np.float32)
    xl = rng.normal(0.5, 2, (rows, cols)).astype(np.float32)
    if rows > 2 and cols > 64:
        xl[1, :32] = 40.0   # a row whose first elements say nothing about its mean (the bf16 kernel's shift estimate)
    try:
        T.tune("layernorm", 0, 0, 0, 4)
        got32 = T.layernorm_rows(dev_f32(xl, cuda), dev_f32(g32, cuda), dev_f32(b32, cuda), 1e-5).cpu().numpy()
        xb, gb, bb = oracle.f32_to_bf16(xl), oracle.f32_to_bf16(g32), oracle.f32_to_bf16(b32)
        got16 = T.layernorm_rows(dev_bf16(xb, cuda), dev_bf16(gb, cuda), dev_bf16(bb, cuda), 1e-5)
    finally:
        T.tune("layernorm")
    ref32 = T.layernorm_rows(dev_f32(xl, cuda), dev_f32(g32, cuda), dev_f32(b32, cuda), 1e-5).cpu().numpy()
    want = oracle.layernorm_rows_f32(xl, g32, b32, 1e-5)
    assert np.abs(got32 - want).max() <= 2e-5 * max(1.0, np.abs(want).max())
    assert np.abs(got32 - ref32).max() <= 2e-5 * max(1.0, np.abs(want).max())
    assert checks.layernorm_bf16_close(got16.view(torch.int16).cpu().numpy().view(np.uint16), xb, gb, bb)
    assert T.device_status() == 0


@pytest.mark.parametrize("seed", [0, 1, 2])
def test_row_kernels_around_dispatch_boundaries(oracle, cuda, seed):
    # row lengths a few columns either side of every length at which the launchers change kernel or shape, with
    # row counts below, at and above the number of SMs; softmax fp32, layer-norm fp32 and bf16 through the heuristic
    from oracle import checks
    rnd = np.random.default_rng(1000 + seed)
    bounds = [16, 32, 64, 128, 256, 512, 1024, 2048, 4096, 8192, 10240, 12288, 16384, 20480, 24576, 32768, 45056,
              65536, 90112, 131072]
    for _ in range(14):
        cols = max(1, int(rnd.choice(bounds)) + int(rnd.choice([-9, -8, -4, -3, -1, 0, 0, 1, 2, 4, 7, 8, 12, 16])))
        rows = int(rnd.choice([1, 2, 3, 7, 40, 147, 148, 149, 300]))
        rows = max(1, min(rows, (1 << 21) // cols))
        x = (3 * rnd.normal(0, 1, (rows, cols)) + rnd.choice([0.0, 0.5, -2.0])).astype(np.float32)
        g = rnd.normal(1, 0.1, cols).astype(np.float32)
        b = rnd.normal(0, 0.1, cols).astype(np.float32)
        what = f"rows {rows} cols {cols}"
        got = T.softmax_rows(dev_f32(x, cuda)).cpu().numpy()
        assert checks.softmax_close(got, x), "softmax " + what
        got = T.layernorm_rows(dev_f32(x, cuda), dev_f32(g, cuda), dev_f32(b, cuda), 1e-5).cpu().numpy()
        want = oracle.layernorm_rows_f32(x, g, b, 1e-5)
        x64 = x.astype(np.float64)
        y64 = (x64 - x64.mean(1, keepdims=True)) / np.sqrt(x64.var(1, keepdims=True) + 1e-5) * g + b
        scale = np.abs(y64).max()
        assert np.abs(got - y64).max() <= 1e-5 * scale, "layernorm f32 " + what
        assert np.abs(got - want).max() <= 1e-5 * scale + np.abs(want - y64).max(), "layernorm f32 vs oracle " + what
        xb, gb, bb = oracle.f32_to_bf16(x), oracle.f32_to_bf16(g), oracle.f32_to_bf16(b)
        got16 = host_bits(T.layernorm_rows(dev_bf16(xb, cuda), dev_bf16(gb, cuda), dev_bf16(bb, cuda), 1e-5))
        assert checks.layernorm_bf16_close(got16, xb, gb, bb), "layernorm bf16 " + what
    assert T.device_status() == 0


# (1, 66305, 64) and (1, 150000, 128): reduced extents for which rounding the range length up leaves fewer
# ranges than CTAs were wanted (the plan must not hand a CTA a range that starts past the end of k)
@pytest.mark.parametrize("nb,nk,nc", [(1, 50000, 64), (2, 7001, 100), (1, 4096, 33), (3, 600, 260),
                                      (1, 66305, 64), (1, 150000, 128)])
def test_chain_outer_k_split_over_ctas(oracle, cuda, nb, nk, nc):
    # middle-axis lambda chains with few columns and a long k: k ranges over CTAs + the finishing kernel
    rng = np.random.default_rng(nk)
    x = rng.uniform(-1, 1, (nb, nk, nc)).astype(np.float32)
    z = rng.uniform(-1, 1, (nb, nk, nc)).astype(np.float32)
    xd, zd = dev_f32(x, cuda), dev_f32(z, cuda)
    n0 = T.launch_count()
    got = T.chain_reduce([xd, zd], "p0 * p1", axis=1).cpu().numpy()          # ahead-of-time lambda
    assert T.launch_count() - n0 == 2
    want = (x.astype(np.float64) * z).sum(1)
    assert (np.abs(got - want) <= 1e-5 * np.abs(x.astype(np.float64) * z).sum(1)).all()
    n0 = T.launch_count()
    got = T.chain_reduce([xd], "expf(p0) * 0.5f", axis=1, post_expr="p0 + 1.0f").cpu().numpy()   # run-time compiled
    assert T.launch_count() - n0 == 2
    want = (np.exp(x.astype(np.float64)) * 0.5).sum(1) + 1.0
    assert (np.abs(got - want) <= 2e-5 * np.abs(want)).all()
    got = T.chain_reduce([xd], "p0", combine_expr="fmaxf(p0, p1)", init=-np.inf, axis=1).cpu().numpy()
    assert np.array_equal(got, x.max(1))                                       # order-independent: bit-exact
    # init enters exactly once, whatever the number of ranges
    got = T.chain_reduce([xd, zd], "p0 * p1", axis=1, init=100.0).cpu().numpy()
    want = (x.astype(np.float64) * z).sum(1) + 100.0
    assert (np.abs(got - want) <= 1e-5 * (np.abs(x.astype(np.float64) * z).sum(1) + 100.0)).all()


def test_chain_outer_generic(oracle, cuda):
    rng = np.random.default_rng(31)
    x = rng.normal(0, 2, (5, 61, 70)).astype(np.float32)
    got = T.chain_reduce([dev_f32(x, cuda)], "p0", combine_expr="fmaxf(p0, p1)", init=-np.inf, axis=1).cpu().numpy()
    assert np.array_equal(got, x.max(1))
    got0 = T.chain_reduce([dev_f32(x, cuda)], "p0", axis=0).cpu().numpy()
    assert np.abs(got0 - x.sum(0)).max() <= 1e-5 * np.abs(x).sum(0).max()


# ----------------------------------------------------------------------------
# errors reach the caller as status codes, never as a device fault
# ----------------------------------------------------------------------------
def test_errors_through_the_python_host(cuda):
    x = torch.zeros((4, 8), device=cuda)
    with pytest.raises(T.TcabError) as e:
        T.softmax_rows(x, out=torch.zeros((4, 9), device=cuda))
    assert e.value.status == T._lib.ERR_SHAPE
    with pytest.raises(ValueError, match="contiguous"):
        T.softmax_rows(x.t())
    with pytest.raises(T.TcabError) as e:
        T.chain_reduce([x], "p0", combine_expr="(p0 * p1)")  # a product reducer has no kernel
    assert e.value.status == T._lib.ERR_UNSUPPORTED
    n0 = T.launch_count()
    T.softmax_rows(x)
    assert T.launch_count() == n0 + 1


# ----------------------------------------------------------------------------
# contraction with fused bias + ReLU (bf16 in, fp32 accumulate, bf16 out)
# ----------------------------------------------------------------------------
def gemm_inputs(oracle, m, k, n, seed):
    rng = np.random.default_rng(seed)
    sc = 1.0 / np.sqrt(max(k, 1))
    a = oracle.f32_to_bf16((rng.normal(0, 1, (m, k)) * sc).astype(np.float32))
    b = oracle.f32_to_bf16((rng.normal(0, 1, (k, n)) * sc).astype(np.float32))
    bias = rng.normal(0, 0.02, n).astype(np.float32)
    return a, b, bias


def rel_frobenius(got, want):
    return np.linalg.norm(got.astype(np.float64) - want) / max(np.linalg.norm(want), 1e-30)


@pytest.mark.parametrize("m,k,n", [(256, 64, 256), (128, 128, 64), (256, 512, 256), (300, 200, 520), (1, 8, 8),
                                   (513, 1032, 264), (1024, 2048, 1536)])
@pytest.mark.parametrize("act", ["relu", "none"])
def test_gemm_bias_act(oracle, cuda, m, k, n, act):
    a, b, bias = gemm_inputs(oracle, m, k, n, m * 7 + k * 3 + n)
    want = oracle.bf16_to_f32(oracle.gemm_bias_act_bf16(a, b, bias, act))
    buf, out = guarded((m, n), torch.bfloat16, cuda)
    T.gemm_bias_act(dev_bf16(a, cuda), dev_bf16(b, cuda), dev_f32(bias, cuda), act, out=out)
    got = out.float().cpu().numpy()
    check_guards(buf, torch.bfloat16)
    assert T.device_status() == 0
    assert (got != torch.tensor(CANARY).to(torch.bfloat16).float().item()).all()
    assert rel_frobenius(got, want) <= 1e-3  # bf16-in / fp32-accumulate contraction: relative Frobenius error
    # element-wise: one bf16 ulp of the value plus the fp32 accumulation error of k products
    assert (np.abs(got - want) <= 2.0 ** -7 * np.abs(want) + 1e-5 * np.sqrt(k)).all()


@pytest.mark.parametrize("seed", [0, 1])
def test_gemm_shapes_around_kernel_selection(oracle, cuda, seed):
    # M, N, K either side of what the launcher switches on: one 128-row band or more, fewer or more 256 x 256 tiles
    # than half the SMs, K long enough for one, two or more K ranges; ragged edges in every dimension
    rnd = np.random.default_rng(500 + seed)
    ms = [1, 64, 128, 129, 256, 300, 512, 1100, 2304]
    ns = [8, 120, 256, 264, 520, 1024, 2304]
    ks = [8, 72, 1024, 2048, 2056, 4096, 8192]
    done = 0
    while done < 12:
        m, n, k = int(rnd.choice(ms)), int(rnd.choice(ns)), int(rnd.choice(ks))
        if m * n * k > 3e8:
            continue
        done += 1
        act = "relu" if done % 2 else "none"
        a, b, bias = gemm_inputs(oracle, m, k, n, m + 3 * n + 7 * k)
        want = oracle.bf16_to_f32(oracle.gemm_bias_act_bf16(a, b, bias, act))
        buf, out = guarded((m, n), torch.bfloat16, cuda)
        T.gemm_bias_act(dev_bf16(a, cuda), dev_bf16(b, cuda), dev_f32(bias, cuda), act, out=out)
        got = out.float().cpu().numpy()
        check_guards(buf, torch.bfloat16)
        what = f"m {m} n {n} k {k} {act}"
        assert rel_frobenius(got, want) <= 1e-3, what
        assert (np.abs(got - want) <= 2.0 ** -7 * np.abs(want) + 1e-5 * np.sqrt(k)).all(), what
    assert T.device_status() == 0


@pytest.mark.parametrize("m,k,n", [(512, 64, 256), (300, 200, 520), (1024, 2048, 1536), (1, 8, 8)])
@pytest.mark.parametrize("variant", [2, 3, 4])
def test_gemm_cta_pair_variant(oracle, cuda, m, k, n, variant):
    # the kernels behind the tuning hook: 2 = cta_group::2 (clusters of two CTAs, M = 256 per MMA, 512 x 256 tiles),
    # 3 = double-buffered accumulators on 128 x 256 tiles, 4 = the same on CTA pairs (256 x 256 tiles)
    a, b, bias = gemm_inputs(oracle, m, k, n, m + k + n)
    want = oracle.bf16_to_f32(oracle.gemm_bias_act_bf16(a, b, bias, "relu"))
    buf, out = guarded((m, n), torch.bfloat16, cuda)
    try:
        T.tune("gemm", 0, variant, 0, 1)  # the kernel variant alone: no K split
        T.gemm_bias_act(dev_bf16(a, cuda), dev_bf16(b, cuda), dev_f32(bias, cuda), "relu", out=out)
        single_off = out.float().cpu().numpy()
    finally:
        T.tune("gemm")
    check_guards(buf, torch.bfloat16)
    assert T.device_status() == 0
    assert rel_frobenius(single_off, want) <= 1e-3
    # both kernels accumulate every output over ascending k in the tensor core: identical bits (with the K split
    # switched off: its partial sums round differently)
    try:
        T.tune("gemm", 0, 0, 0, 1)
        ref = T.gemm_bias_act(dev_bf16(a, cuda), dev_bf16(b, cuda), dev_f32(bias, cuda), "relu").float().cpu().numpy()
    finally:
        T.tune("gemm")
    assert np.array_equal(single_off, ref)


@pytest.mark.parametrize("m,k,n,variant,ranges", [(100, 4096, 512, 0, 0), (300, 2048, 264, 0, 0), (16, 8192, 1024, 0, 0),
                                                     (130, 200, 264, 3, 3), (260, 1032, 520, 4, 5), (128, 64, 256, 3, 4),
                                                     (513, 4096, 776, 4, 2)])
def test_gemm_k_split(oracle, cuda, m, k, n, variant, ranges):
    # few output tiles and a long K: ranges of K blocks become units of work. Three forms add the ranges, the bias and
    # the activation, all in ascending order and so with identical bits: (a) the CTAs of a cluster hold one range of a
    # 128-row tile each, exchange the rows they do not own through an L2-resident workspace and add their own rows
    # after a cluster barrier, one launch (the library's choice while every cluster is resident at once, or tuning
    # value p1 = 5); (b) p2 = 32: every fp32 partial goes to the workspace and a second kernel adds them; (c) p2 = 16:
    # the epilogue warp that arrives last at a block of the tile adds them inside the one launch (measured slower,
    # kept for comparison). variant / ranges = 0: the library's own choice.
    a, b, bias = gemm_inputs(oracle, m, k, n, m + 3 * k + n)
    want = oracle.bf16_to_f32(oracle.gemm_bias_act_bf16(a, b, bias, "relu"))
    buf, out = guarded((m, n), torch.bfloat16, cuda)
    n0 = T.launch_count()
    try:
        if variant:
            T.tune("gemm", 0, variant, 0, ranges)
        T.gemm_bias_act(dev_bf16(a, cuda), dev_bf16(b, cuda), dev_f32(bias, cuda), "relu", out=out)
    finally:
        T.tune("gemm")
    launches = T.launch_count() - n0
    got = out.float().cpu().numpy()
    check_guards(buf, torch.bfloat16)
    assert T.device_status() == 0
    split = variant == 0 or min(ranges, (k + 63) // 64) > 1
    if split:
        assert launches == (1 if variant == 0 else 2), "a cluster per tile, or the contraction and the finishing kernel"
    assert rel_frobenius(got, want) <= 1e-3
    # the three forms over the SAME ranges (the library's own choice of their number differs between the forms)
    r = ranges or 4
    kernel = variant or (3 if m <= 128 else 4)
    split_r = min(r, (k + 63) // 64) > 1
    same = None
    for p1, p2, expect in [(kernel, 32, 2 if split_r else 1), (kernel, 16, 1), (5, 0, 1)]:
        try:             # each form three times: the arrival counters of (c) return to zero
            T.tune("gemm", 0, p1, p2, r)
            for _ in range(3):
                buf, out = guarded((m, n), torch.bfloat16, cuda)
                n0 = T.launch_count()
                T.gemm_bias_act(dev_bf16(a, cuda), dev_bf16(b, cuda), dev_f32(bias, cuda), "relu", out=out)
                assert T.launch_count() - n0 == expect, (p1, p2)
                check_guards(buf, torch.bfloat16)
                bits = out.float().cpu().numpy()
                same = bits if same is None else same
                assert np.array_equal(bits, same), (p1, p2)
        finally:
            T.tune("gemm")
    if variant:
        assert np.array_equal(same, got)
    assert T.device_status() == 0
    assert (np.abs(got - want) <= 2.0 ** -7 * np.abs(want) + 1e-5 * np.sqrt(k)).all()
    # no bias, no activation through the same path
    want2 = oracle.bf16_to_f32(oracle.gemm_bias_act_bf16(a, b, None, "none"))
    try:
        if variant:
            T.tune("gemm", 0, variant, 0, ranges)
        got2 = T.gemm_bias_act(dev_bf16(a, cuda), dev_bf16(b, cuda), None, "none").float().cpu().numpy()
    finally:
        T.tune("gemm")
    assert rel_frobenius(got2, want2) <= 1e-3


def test_gemm_without_bias_and_empty_k(oracle, cuda):
    a, b, bias = gemm_inputs(oracle, 256, 128, 256, 5)
    want = oracle.bf16_to_f32(oracle.gemm_bias_act_bf16(a, b, None, "none"))
    got = T.gemm_bias_act(dev_bf16(a, cuda), dev_bf16(b, cuda), None, "none").float().cpu().numpy()
    assert rel_frobenius(got, want) <= 1e-3
    # K = 0: an empty reduction returns init = 0, so c = act(bias) (design/tca.md:299)
    a0 = torch.zeros((64, 0), device=cuda, dtype=torch.bfloat16)
    b0 = torch.zeros((0, 64), device=cuda, dtype=torch.bfloat16)
    c0 = T.gemm_bias_act(a0, b0, dev_f32(bias[:64], cuda), "relu").float().cpu().numpy()
    want0 = oracle.bf16_to_f32(oracle.f32_to_bf16(np.maximum(bias[:64], 0)))
    assert np.array_equal(c0, np.broadcast_to(want0, (64, 64)))


@pytest.mark.parametrize("m,n,k", [(4000, 5000, 3000), (4096, 2440, 256), (2304, 2184, 1024), (4096, 5064, 512)])
def test_gemm_large_ragged_shapes_exact_on_small_integers(cuda, m, n, k):
    """Many 256 x 256 tiles with ragged edges in every dimension, small integers so that every element is exact: the
    last tile column holds boxes that start inside N followed by boxes that lie outside (N = 256 j + 136, + 184: a
    warp's staging buffers must not be refilled while a store of the previous box still reads them)."""
    gen = torch.Generator(device=cuda).manual_seed(m + n + k)
    a = torch.randint(-2, 3, (m, k), generator=gen, device=cuda).to(torch.bfloat16)
    b = torch.randint(-2, 3, (k, n), generator=gen, device=cuda).to(torch.bfloat16)
    bias = torch.randint(-4, 5, (n,), generator=gen, device=cuda).float()
    want = (a.float() @ b.float() + bias).to(torch.bfloat16)      # |sums| < 2^24: exact in fp32
    for variant in (0, 1, 0, 1, 4):                                # what the library picks, the 256 x 256 kernel, CTA pairs;
        buf, out = guarded((m, n), torch.bfloat16, cuda)           # more than once: a race does not show every time
        try:
            T.tune("gemm", 0, variant, 0, 1 if variant else 0)
            T.gemm_bias_act(a, b, bias, "none", out=out)
        finally:
            T.tune("gemm")
        check_guards(buf, torch.bfloat16)
        bad = (out != want)
        assert not bool(bad.any()), f"variant {variant}: {int(bad.sum())} mismatches, first at {bad.nonzero()[0].tolist()}"
    assert T.device_status() == 0


def test_gemm_exact_on_small_integers(oracle, cuda):
    # products and sums of small integers are exact in bf16/fp32: every accumulation order agrees bit for bit
    rng = np.random.default_rng(3)
    m, k, n = 512, 256, 512
    a = oracle.f32_to_bf16(rng.integers(-2, 3, (m, k)).astype(np.float32))
    b = oracle.f32_to_bf16(rng.integers(-2, 3, (k, n)).astype(np.float32))
    bias = rng.integers(-4, 5, n).astype(np.float32)
    want = oracle.gemm_bias_act_bf16(a, b, bias, "relu")
    got = host_bits(T.gemm_bias_act(dev_bf16(a, cuda), dev_bf16(b, cuda), dev_f32(bias, cuda), "relu"))
    assert np.array_equal(got, want)


def test_gemm_full_size_rows_of_every_band_and_linearity(oracle, cuda, parity_counts):
    # the benchmark configuration: 8192^3, a,b ~ N(0,1)/sqrt(8192), bias ~ N(0,0.02)
    gen = torch.Generator(device=cuda).manual_seed(11)
    sc = 1.0 / np.sqrt(8192)
    a = (torch.randn((8192, 8192), generator=gen, device=cuda) * sc).to(torch.bfloat16)
    b = (torch.randn((8192, 8192), generator=gen, device=cuda) * sc).to(torch.bfloat16)
    bias = torch.randn((8192,), generator=gen, device=cuda) * 0.02
    c = T.gemm_bias_act(a, b, bias, "relu")
    assert T.device_status() == 0
    # two rows of each of the 64 bands of 128 rows (one per 64-row half, at varying offsets) and the last row,
    # all 8192 columns each: every CTA's tile rows, both accumulators and every column box are sampled
    # (testing/runners/gemm.cu:44-56 is the loop the oracle restates)
    picks = sorted({band * 128 + (band * 37) % 64 for band in range(64)} |
                   {band * 128 + 64 + (band * 11) % 64 for band in range(64)} | {8191})
    rows = torch.tensor(picks, device=cuda)
    want = oracle.bf16_to_f32(oracle.gemm_bias_act_bf16(host_bits(a[rows]), host_bits(b), bias.cpu().numpy(), "relu"))
    got = c[rows].float().cpu().numpy()
    assert rel_frobenius(got, want) <= 1e-3
    per_row = np.linalg.norm(got - want, axis=1) / np.maximum(np.linalg.norm(want, axis=1), 1e-30)
    assert per_row.max() <= 1e-3, (picks[int(per_row.argmax())], per_row.max())   # no single bad row hides in the norm
    parity_counts["C5 contraction bf16 8192^3"] = {"rows_checked": len(picks), "elements": int(got.size),
                                                   "rel_frobenius": float(rel_frobenius(got, want)),
                                                   "worst_row_rel": float(per_row.max())}
    # linearity without the epilogue: (2a) @ b == 2 (a @ b) exactly (scaling by 2 is exact in bf16 and fp32)
    c1 = T.gemm_bias_act(a, b, None, "none")
    c2 = T.gemm_bias_act(a * 2, b, None, "none")
    assert torch.equal(c2.float(), c1.float() * 2)


# ----------------------------------------------------------------------------
# long rows split over several CTAs (partials through the library's scratch buffer)
# ----------------------------------------------------------------------------
@pytest.mark.parametrize("rows,cols", [(1, 1 << 20), (2, 70001), (3, 262144), (7, 1000003), (100, 40000)])
def test_split_reduction_long_rows(oracle, cuda, rows, cols):
    from oracle import checks
    rng = np.random.default_rng(rows + cols)
    x = rng.uniform(-1, 1, (rows, cols)).astype(np.float32)
    xd = dev_f32(x, cuda)
    n0 = T.launch_count()
    got = T.chain_reduce([xd], "(0.5f*p0 + 0.25f) * (0.5f*p0 + 0.25f)").cpu().numpy()
    assert T.launch_count() - n0 == 2  # the split pass and the finishing pass
    assert checks.rowsum_close(got, x)
    # max is order-independent: bit-exact whatever the split, and init takes part exactly once
    gm = T.chain_reduce([xd], "p0", combine_expr="fmaxf(p0, p1)", init=0.5).cpu().numpy()
    assert np.array_equal(gm, np.maximum(x.max(1), np.float32(0.5)))
    # the same rows with the split switched off agree to rounding; with a forced odd split as well
    try:
        T.tune("reduce_inner", 0, 1)
        one = T.chain_reduce([xd], "(0.5f*p0 + 0.25f) * (0.5f*p0 + 0.25f)").cpu().numpy()
        T.tune("reduce_inner", 0, 7)
        odd = T.chain_reduce([xd], "(0.5f*p0 + 0.25f) * (0.5f*p0 + 0.25f)").cpu().numpy()
    finally:
        T.tune("reduce_inner")
    assert checks.rowsum_close(one, x) and checks.rowsum_close(odd, x)


def test_split_reduction_with_piped_map_and_two_operands(oracle, cuda):
    rng = np.random.default_rng(17)
    x = rng.uniform(0, 1, (2, 300000)).astype(np.float32)
    z = rng.uniform(0, 1, (2, 300000)).astype(np.float32)
    got = T.chain_reduce([dev_f32(x, cuda), dev_f32(z, cuda)], "(p0 * p0) * p1", post_expr="p0 * rsqrtf(p0 * c0 + c1)",
                         captures=(1.0 / 300000, 1e-5)).cpu().numpy()
    s = ((x.astype(np.float64) ** 2) * z).sum(1)
    want = s / np.sqrt(s / 300000 + 1e-5)
    assert np.abs(got - want).max() <= 1e-5 * np.abs(want).max()


# ----------------------------------------------------------------------------
# lambdas without an ahead-of-time kernel: compiled at run time from the same kernel text
# ----------------------------------------------------------------------------
JIT_SUITE = {
    # testing/kernels/dedup/dup_expr.tca and dup_const.tca, lambdas as the .tca files spell them
    "dup_expr": ("((p0*p0 + p0*p0) * c0 + (p0*p0 + p0*p0) * c1) * p1", (1.5, 0.25), 1e-5),
    "dup_const": ("(0.5f * (p0 + 0.5f * p0 * p0) * (1.0f + 0.044715f * p0) + tanhf(0.79788456f * (p0 + 0.044715f * p0)"
                  " + 0.79788456f * 0.5f * p0) * (1.0f - 0.5f)) * p1", (), 1e-5),
}


@pytest.mark.parametrize("name", sorted(JIT_SUITE))
def test_reference_suite_kernels_compiled_at_run_time(oracle, cuda, name):
    expr, caps, tol = JIT_SUITE[name]
    x, z = oracle.suite_inputs(name)
    want = oracle.suite(name)
    buf, out = guarded(want.shape, torch.float32, cuda)
    T.chain_reduce([dev_f32(x, cuda), dev_f32(z, cuda)], expr, captures=caps, axis=2, out=out)
    got = out.cpu().numpy()
    check_guards(buf, torch.float32)
    assert (got == CANARY).sum() == 0
    assert np.abs(got.astype(np.float64) - want).max() <= tol
    g = GOLDEN[name]
    assert abs(got.astype(np.float64).sum() - g["checksum"]) <= 1e-5 * abs(g["checksum"])


def test_run_time_compiled_lambdas_every_kernel_shape(oracle, cuda):
    rng = np.random.default_rng(41)
    expr, post = "sinf(p0) * cosf(p1) + c0", "sqrtf(fabsf(p0)) - c1"
    f = lambda a, b: np.sin(a.astype(np.float64)) * np.cos(b.astype(np.float64)) + 0.5  # noqa: E731
    # innermost axis at every group size, vector and scalar paths, the split path, and a middle axis
    for shape, axis in [((300, 8), 1), ((50, 200), 1), ((20, 3000), 1), ((6, 20000), 1), ((9, 77), 1),
                        ((2, 400000), 1), ((5, 40, 260), 1), ((3, 33, 50), 1), ((4, 10, 6), 0)]:
        a = rng.uniform(-2, 2, shape).astype(np.float32)
        b = rng.uniform(-2, 2, shape).astype(np.float32)
        got = T.chain_reduce([dev_f32(a, cuda), dev_f32(b, cuda)], expr, post_expr=post, captures=(0.5, 0.25),
                             axis=axis).cpu().numpy()
        want = np.sqrt(np.abs(f(a, b).sum(axis))) - 0.25
        scale = np.abs(f(a, b)).sum(axis)
        assert (np.abs(got - want) <= 2e-5 * np.sqrt(scale) + 1e-5).all(), (shape, axis)
    # max and min combiners, bit-exact against numpy on an exactly representable map
    a = rng.integers(-50, 50, (17, 513)).astype(np.float32)
    got = T.chain_reduce([dev_f32(a, cuda)], "p0 * 0.5f - 3.0f", combine_expr="fminf(p0, p1)", init=np.inf).cpu().numpy()
    assert np.array_equal(got, (a * 0.5 - 3.0).min(1).astype(np.float32))
    # a lambda the validator refuses never reaches the compiler
    with pytest.raises(T.TcabError) as e:
        T.chain_reduce([dev_f32(a, cuda)], "p0); } __global__ void k() { (void)(0")
    assert e.value.status == T._lib.ERR_INVALID_ARG
    # the entry point that allocates nothing runs compiled lambdas too, but never compiles one itself
    # (loading a code image allocates device memory): an unknown lambda is refused until it has been prepared
    out = torch.empty((17,), device=cuda)
    with pytest.raises(T.TcabError) as e:
        T.chain_reduce_noalloc([dev_f32(a, cuda)], "cosf(p0) * cosf(p0)", out=out)
    assert e.value.status == T._lib.ERR_UNSUPPORTED and "tcab_chain_prepare" in e.value.message
    T.chain_prepare("cosf(p0) * cosf(p0)", n_ins=1)
    T.chain_reduce_noalloc([dev_f32(a, cuda)], "cosf(p0) * cosf(p0)", out=out)
    assert np.allclose(out.cpu().numpy(), (np.cos(a.astype(np.float64)) ** 2).sum(1), rtol=1e-5)


# ----------------------------------------------------------------------------
# the reference's matmul-shaped suite kernels: fp32 contraction chains
# ----------------------------------------------------------------------------
GELU = "0.5f*p0*(1.0f + tanhf(0.79788456f*(p0 + 0.044715f*p0*p0*p0)))"   # testing/kernels/fusion/mlp.tca
CONTRACT_SUITE = {
    # name: (rhs_is_nk, post, captures)  -- tolerance 2e-3 for all of them (testing/suite.toml)
    "mm_small": (False, None, ()), "mm_mid": (False, None, ()), "mm_splitk": (False, None, ()),
    "gemm": (False, None, ()), "mlp": (False, GELU, ()), "qk_score": (True, "p0 * c0", (0.125,)),
}


@pytest.mark.parametrize("name", sorted(CONTRACT_SUITE))
def test_reference_suite_contractions(oracle, cuda, name):
    nk, post, caps = CONTRACT_SUITE[name]
    x, z = oracle.suite_inputs(name)
    want = oracle.suite(name)
    buf, out = guarded(want.shape, torch.float32, cuda)
    T.chain_contract(dev_f32(x, cuda), dev_f32(z, cuda), "(p0 * p1)", rhs_is_nk=nk, post_expr=post, captures=caps,
                     out=out)
    got = out.cpu().numpy()
    check_guards(buf, torch.float32)
    assert (got == CANARY).sum() == 0
    assert np.abs(got.astype(np.float64) - want).max() <= 2e-3
    g = GOLDEN[name]
    assert abs(got.astype(np.float64).sum() - g["checksum"]) <= 1e-5 * abs(g["checksum"])


def test_e2e_matmul_scale_fixture(oracle, cuda):
    # internal/e2e/frontend_test.go:33-34,194-209: 64 x 128 x 64, scale 1.5, tolerance 2e-3
    a = oracle.elem_fill(64 * 128).reshape(64, 128)
    b = oracle.elem_fill(128 * 64).reshape(128, 64)
    got = T.chain_contract(dev_f32(a, cuda), dev_f32(b, cuda), post_expr="p0 * c0", captures=(1.5,)).cpu().numpy()
    assert np.abs(got - oracle.matmul_scale_f32(a, b, 1.5)).max() <= 2e-3
    g = GOLDEN["e2e_matmul_scale_64x128x64"]
    assert abs(got.astype(np.float64).sum() - g["checksum"]) <= 1e-5 * g["checksum"]


def test_contraction_ragged_and_other_combiners(oracle, cuda):
    rng = np.random.default_rng(23)
    for m, k, n in [(1, 1, 1), (65, 17, 130), (200, 300, 7), (64, 0, 64)]:
        a = rng.normal(0, 1, (m, k)).astype(np.float32)
        b = rng.normal(0, 1, (k, n)).astype(np.float32)
        got = T.chain_contract(dev_f32(a, cuda), dev_f32(b, cuda)).cpu().numpy()
        want = oracle.matmul_scale_f32(a, b, 1.0) if k else np.zeros((m, n), np.float32)
        assert np.abs(got - want).max() <= 1e-5 * max(1.0, np.abs(want).max())
        gt = T.chain_contract(dev_f32(a, cuda), dev_f32(np.ascontiguousarray(b.T), cuda), rhs_is_nk=True).cpu().numpy()
        assert np.abs(gt - want).max() <= 1e-5 * max(1.0, np.abs(want).max())
    # a max-plus contraction (tropical product): out[m,n] = max_k (a[m,k] + b[k,n]), order-independent
    a = rng.integers(-9, 9, (70, 33)).astype(np.float32)
    b = rng.integers(-9, 9, (33, 45)).astype(np.float32)
    got = T.chain_contract(dev_f32(a, cuda), dev_f32(b, cuda), "p0 + p1", combine_expr="fmaxf(p0, p1)",
                           init=-np.inf).cpu().numpy()
    assert np.array_equal(got, (a[:, :, None] + b[None, :, :]).max(1))
    with pytest.raises(T.TcabError) as e:
        T.chain_contract(dev_f32(a, cuda), dev_f32(a, cuda))
    assert e.value.status == T._lib.ERR_SHAPE and "dim k" in e.value.message


@pytest.mark.parametrize("tile", [4, 8])
def test_contraction_tile_sizes(oracle, cuda, tile):
    # both tile shapes of the fp32 contraction (64 x 64 and 128 x 128 per CTA) on the same inputs: ragged edges in
    # m, n and k, row pitches that allow 16-byte loads and ones that do not, both layouts of rhs, a JIT lambda
    rng = np.random.default_rng(tile)
    try:
        T.tune("gemm", 0, 0, tile)
        for m, k, n in [(129, 16, 257), (300, 203, 130), (255, 64, 128), (128, 37, 131), (1, 5, 300), (260, 48, 9)]:
            a = rng.normal(0, 1, (m, k)).astype(np.float32)
            b = rng.normal(0, 1, (k, n)).astype(np.float32)
            want = oracle.matmul_scale_f32(a, b, 1.0)
            buf, out = guarded((m, n), torch.float32, cuda)
            T.chain_contract(dev_f32(a, cuda), dev_f32(b, cuda), out=out)
            check_guards(buf, torch.float32)
            assert np.abs(out.cpu().numpy() - want).max() <= 1e-5 * np.sqrt(k) * max(1.0, np.abs(want).max())
            gt = T.chain_contract(dev_f32(a, cuda), dev_f32(np.ascontiguousarray(b.T), cuda), rhs_is_nk=True).cpu().numpy()
            assert np.abs(gt - want).max() <= 1e-5 * np.sqrt(k) * max(1.0, np.abs(want).max())
        # a lambda outside the ahead-of-time table (run-time compiled) with a piped map, on a size that needs both
        a = rng.uniform(0, 1, (300, 100)).astype(np.float32)
        b = rng.uniform(0, 1, (100, 200)).astype(np.float32)
        got = T.chain_contract(dev_f32(a, cuda), dev_f32(b, cuda), "p0 * p1 + 0.5f", post_expr="sqrtf(p0)").cpu().numpy()
        want = np.sqrt((a[:, :, None].astype(np.float64) * b[None, :, :] + 0.5).sum(1))
        assert np.abs(got - want).max() <= 1e-5 * np.abs(want).max()
        # operands that start 4 bytes into an allocation: the scalar load path
        big_a = torch.zeros(128 * 64 + 1, device=cuda)
        av = big_a[1:].view(128, 64)
        av.copy_(torch.from_numpy(rng.normal(0, 1, (128, 64)).astype(np.float32)))
        bb = rng.normal(0, 1, (64, 128)).astype(np.float32)
        got = T.chain_contract(av, dev_f32(bb, cuda)).cpu().numpy()
        want = oracle.matmul_scale_f32(av.cpu().numpy(), bb, 1.0)
        assert np.abs(got - want).max() <= 1e-4 * max(1.0, np.abs(want).max())
    finally:
        T.tune("gemm")


# ----------------------------------------------------------------------------
# innermost-axis chains and row kernels on short rows (1 to 32 vectors)
# ----------------------------------------------------------------------------
@pytest.mark.parametrize("rows,cols", [(5000, 4), (3001, 8), (2049, 12), (1500, 16), (1024, 20), (4000, 32), (1111, 36),
                                       (2000, 64), (1300, 100), (1025, 128), (1024, 124), (1100, 132), (1500, 256),
                                       (1027, 300), (1200, 512), (1030, 508)])
def test_short_rows(oracle, cuda, rows, cols):
    rng = np.random.default_rng(rows + cols)
    x = rng.uniform(-1, 1, (rows, cols)).astype(np.float32)
    z = rng.uniform(0, 1, (rows, cols)).astype(np.float32)
    xd, zd = dev_f32(x, cuda), dev_f32(z, cuda)
    x64 = x.astype(np.float64)
    # the benchmark's chain (a table lambda), every row against the oracle and fp64
    buf, out = guarded((rows,), torch.float32, cuda)
    T.chain_reduce([xd], "(0.5f * p0 + 0.25f) * (0.5f * p0 + 0.25f)", axis=1, out=out)
    got = out.cpu().numpy()
    check_guards(buf, torch.float32)
    from oracle import checks
    assert checks.rowsum_close(got, x)
    try:        # a warp per row: the same sums in another order
        T.tune("reduce_inner", 32)
        old = T.chain_reduce([xd], "(0.5f * p0 + 0.25f) * (0.5f * p0 + 0.25f)", axis=1).cpu().numpy()
    finally:
        T.tune("reduce_inner")
    assert (np.abs(got - old) <= 2e-5 * np.abs(old) + 1e-30).all()
    if cols <= 64:   # up to 16 vectors a thread folds its row in ascending order, the reference's: the same BITS as the
        try:         # kernel that gives a thread a row without the coalesced copy, and as the sequential oracle
            T.tune("reduce_inner", 1)
            seq = T.chain_reduce([xd], "(0.5f * p0 + 0.25f) * (0.5f * p0 + 0.25f)", axis=1).cpu().numpy()
        finally:
            T.tune("reduce_inner")
        assert np.array_equal(got, seq)
    # max with init and a piped map: bit-exact
    got = T.chain_reduce([xd], "p0", combine_expr="fmaxf(p0, p1)", init=0.25, axis=1, post_expr="p0 + 1.0f").cpu().numpy()
    assert np.array_equal(got, np.maximum(x.max(1), np.float32(0.25)) + np.float32(1))
    # run-time compiled, two operands, one of them bf16
    zb = oracle.f32_to_bf16(z)
    got = T.chain_reduce([xd, dev_bf16(zb, cuda)], "expf(p0) * f32(p1)", axis=1).cpu().numpy()
    want = (np.exp(x64) * oracle.bf16_to_f32(zb)).sum(1)
    assert (np.abs(got - want) <= 1e-5 * want + 1e-30).all()
    # softmax and layer-norm of the same rows (one, two or four threads per row up to four vectors)
    buf, out = guarded((rows, cols), torch.float32, cuda)
    T.softmax_rows(dev_f32(4 * x, cuda), out=out)
    check_guards(buf, torch.float32)
    assert_softmax_close(out.cpu().numpy(), oracle.softmax_rows(4 * x), 4 * x)
    g = rng.normal(1, 0.1, cols).astype(np.float32)
    b = rng.normal(0, 0.1, cols).astype(np.float32)
    buf, out = guarded((rows, cols), torch.float32, cuda)
    T.layernorm_rows(xd, dev_f32(g, cuda), dev_f32(b, cuda), 1e-5, out=out)
    check_guards(buf, torch.float32)
    y64 = (x64 - x64.mean(1, keepdims=True)) / np.sqrt(x64.var(1, keepdims=True) + 1e-5) * g + b
    assert np.abs(out.cpu().numpy() - y64).max() <= 1e-5 * np.abs(y64).max()
    if cols % 8 == 0:
        xb, gb, bb = oracle.f32_to_bf16(x), oracle.f32_to_bf16(g), oracle.f32_to_bf16(b)
        buf, outb = guarded((rows, cols), torch.bfloat16, cuda)
        T.layernorm_rows(dev_bf16(xb, cuda), dev_bf16(gb, cuda), dev_bf16(bb, cuda), 1e-5, out=outb)
        check_guards(buf, torch.bfloat16)
        assert_layernorm_bf16_close(oracle, host_bits(outb), oracle.layernorm_rows_bf16(xb, gb, bb, 1e-5), xb, gb, bb)


# ----------------------------------------------------------------------------
# rows of 3 * 2^k and 5 * 2^k vectors: register shapes with three and five slots per thread
# ----------------------------------------------------------------------------
@pytest.mark.parametrize("cols", [160, 192, 320, 384, 640, 768, 1280, 1536, 2560, 3072, 5120, 6144])
def test_rows_of_three_and_five_slots(oracle, cuda, cols):
    rows = 333
    rng = np.random.default_rng(cols)
    x = rng.normal(0, 1, (rows, cols)).astype(np.float32)
    g = rng.normal(1, 0.1, cols).astype(np.float32)
    b = rng.normal(0, 0.1, cols).astype(np.float32)
    x64 = x.astype(np.float64)
    buf, out = guarded((rows, cols), torch.float32, cuda)
    T.softmax_rows(dev_f32(4 * x, cuda), out=out)
    check_guards(buf, torch.float32)
    assert_softmax_close(out.cpu().numpy(), oracle.softmax_rows(4 * x), 4 * x)
    buf, out = guarded((rows, cols), torch.float32, cuda)
    T.layernorm_rows(dev_f32(x, cuda), dev_f32(g, cuda), dev_f32(b, cuda), 1e-5, out=out)
    check_guards(buf, torch.float32)
    y64 = (x64 - x64.mean(1, keepdims=True)) / np.sqrt(x64.var(1, keepdims=True) + 1e-5) * g + b
    assert np.abs(out.cpu().numpy() - y64).max() <= 1e-5 * np.abs(y64).max()
    xb, gb, bb = oracle.f32_to_bf16(x), oracle.f32_to_bf16(g), oracle.f32_to_bf16(b)
    buf, outb = guarded((rows, cols), torch.bfloat16, cuda)
    T.layernorm_rows(dev_bf16(xb, cuda), dev_bf16(gb, cuda), dev_bf16(bb, cuda), 1e-5, out=outb)
    check_guards(buf, torch.bfloat16)
    assert_layernorm_bf16_close(oracle, host_bits(outb), oracle.layernorm_rows_bf16(xb, gb, bb, 1e-5), xb, gb, bb)


# ----------------------------------------------------------------------------
# element counts just below 2^32 (the reference's index type): byte offsets beyond 2^32
# ----------------------------------------------------------------------------
def test_element_counts_just_below_two_to_the_32(cuda):
    free, _ = torch.cuda.mem_get_info(cuda)
    if free < 60 * 2**30:
        pytest.skip("needs 40 GB of free device memory")
    rows, cols = (1 << 20) - 3, 4092                       # 4,290,760,716 elements, 17 GB
    x = torch.empty((rows, cols), device=cuda)
    for lo in range(0, rows, 1 << 16):
        x[lo:lo + (1 << 16)].uniform_(-1, 1)
    s = T.chain_reduce([x], "p0 * p0")
    for lo in range(0, rows, 1 << 17):                     # every row, the last ones included
        ref = (x[lo:lo + (1 << 17)].double() ** 2).sum(1)
        assert bool(((s[lo:lo + (1 << 17)].double() - ref).abs() <= 1e-5 * ref).all())
    y = T.map([x], "p0 * 2.0f + 1.0f")
    assert torch.equal(y[-4096:], x[-4096:] * 2 + 1) and torch.equal(y[:4096], x[:4096] * 2 + 1)
    pr = torch.tensor([0, rows // 2, rows - 2, rows - 1], device=cuda)
    T.softmax_rows(x, out=y)
    ref = torch.softmax(x[pr].double(), dim=1)
    assert bool(((y[pr].double() - ref).abs() <= 2e-5 * ref).all())
    del y
    t = x.view(-1)[:65000 * 256 * 256].view(65000, 256, 256)
    got = T.reduce_outer(t)
    pb = torch.tensor([0, 33333, 64999], device=cuda)
    assert torch.equal(got["max"][pb], t[pb].max(1).values)
    first = (t[pb] == t[pb].max(1, keepdim=True).values).float().argmax(1).int()
    assert torch.equal(got["argmax"][pb], first)
    assert T.device_status() == 0


# ----------------------------------------------------------------------------
# innermost-axis chains on rows that are not whole 16-byte vectors (aligned operands)
# ----------------------------------------------------------------------------
@pytest.mark.parametrize("rows,cols", [(5000, 1), (4001, 2), (3000, 3), (2049, 5), (2500, 7), (1500, 13), (1200, 33),
                                       (1025, 63), (1024, 62), (1100, 65), (1300, 127), (1111, 129), (1030, 255),
                                       (1500, 1023), (1026, 1025), (300, 2563), (200, 4097), (40, 30001), (500, 7),
                                       (33, 3), (7, 129)])
def test_innermost_rows_that_are_not_whole_vectors(oracle, cuda, rows, cols):
    rng = np.random.default_rng(rows + cols)
    x = rng.uniform(-1, 1, (rows, cols)).astype(np.float32)
    z = rng.uniform(0, 1, (rows, cols)).astype(np.float32)
    xd, zd = dev_f32(x, cuda), dev_f32(z, cuda)
    x64 = x.astype(np.float64)
    expr = "(0.5f * p0 + 0.25f) * (0.5f * p0 + 0.25f)"
    buf, out = guarded((rows,), torch.float32, cuda)
    n0 = T.launch_count()
    T.chain_reduce([xd], expr, axis=1, out=out)
    assert T.launch_count() - n0 <= 2          # two when few long rows are split over CTAs
    got = out.cpu().numpy()
    check_guards(buf, torch.float32)
    from oracle import checks
    assert checks.rowsum_close(got, x)
    try:        # the kernels on 4-byte loads: a thread per row (the reference's order), a warp per row
        T.tune("reduce_inner", 1)
        seq = T.chain_reduce([xd], expr, axis=1).cpu().numpy()
        T.tune("reduce_inner", 32)
        old = T.chain_reduce([xd], expr, axis=1).cpu().numpy()
    finally:
        T.tune("reduce_inner")
    assert (np.abs(got - old) <= 2e-5 * np.abs(old) + 1e-30).all()
    if cols <= 64 and rows >= 1024:   # a thread folds its row in ascending order: the same BITS as the sequential kernel
        assert np.array_equal(got, seq)
    # max with init and a piped map: bit-exact
    got = T.chain_reduce([xd], "p0", combine_expr="fmaxf(p0, p1)", init=0.25, axis=1, post_expr="p0 + 1.0f").cpu().numpy()
    assert np.array_equal(got, np.maximum(x.max(1), np.float32(0.25)) + np.float32(1))
    # run-time compiled, two operands, one of them bf16; then three fp32 operands
    zb = oracle.f32_to_bf16(z)
    got = T.chain_reduce([xd, dev_bf16(zb, cuda)], "expf(p0) * f32(p1)", axis=1).cpu().numpy()
    want = (np.exp(x64) * oracle.bf16_to_f32(zb)).sum(1)
    assert (np.abs(got - want) <= 1e-5 * want + 1e-30).all()
    got = T.chain_reduce([xd, zd, xd], "p0 * p1 + p2 * p2", init=2.0, axis=1).cpu().numpy()
    want = (x64 * z + x64 * x64).sum(1) + 2.0
    assert (np.abs(got - want) <= 1e-5 * (np.abs(x64 * z) + x64 * x64).sum(1) + 1e-5).all()


# ----------------------------------------------------------------------------
# middle-axis chains on narrow rows and short reduced axes: a warp per (b, column tile)
# ----------------------------------------------------------------------------
@pytest.mark.parametrize("nb,nk,nc", [(3000, 256, 4), (2500, 300, 8), (1300, 77, 16), (700, 1000, 32), (4000, 4, 1024),
                                      (2000, 8, 256), (900, 33, 64), (5000, 1, 4), (1200, 63, 132), (600, 5, 2052),
                                      (1, 7, 8), (3, 2, 4),
                                      # any number of column groups; rows that are not whole vectors (4-byte loads)
                                      (2000, 256, 12), (1100, 90, 20), (800, 300, 48), (900, 40, 100), (3000, 64, 6),
                                      (1500, 100, 7), (2500, 33, 3), (4000, 17, 1), (700, 8, 2050), (900, 31, 33),
                                      (1200, 200, 31), (5, 3, 2)])
def test_middle_axis_chains_warp_per_tile(oracle, cuda, nb, nk, nc):
    rng = np.random.default_rng(nb + nk + nc)
    x = rng.uniform(-1, 1, (nb, nk, nc)).astype(np.float32)
    z = rng.uniform(0, 1, (nb, nk, nc)).astype(np.float32)
    xd, zd = dev_f32(x, cuda), dev_f32(z, cuda)
    x64 = x.astype(np.float64)
    # a table lambda (compiled ahead of time) with a sum; the kernel that a CTA per tile runs gives the same sums
    buf, out = guarded((nb, nc), torch.float32, cuda)
    n0 = T.launch_count()
    T.chain_reduce([xd], "p0", axis=1, out=out)
    assert T.launch_count() - n0 == 1
    got = out.cpu().numpy()
    check_guards(buf, torch.float32)
    mag = np.abs(x64).sum(1)
    assert (np.abs(got - x64.sum(1)) <= 1e-5 * mag + 1e-30).all()
    try:
        T.tune("reduce_inner", 0, 0, 0, 1)
        old = T.chain_reduce([xd], "p0", axis=1).cpu().numpy()
    finally:
        T.tune("reduce_inner")
    assert (np.abs(got - old) <= 2e-5 * mag + 1e-30).all()
    # max: order-independent, bit-exact; with init and a piped map
    got = T.chain_reduce([xd], "p0", combine_expr="fmaxf(p0, p1)", init=-0.5, axis=1, post_expr="p0 * 2.0f").cpu().numpy()
    assert np.array_equal(got, np.maximum(x.max(1), np.float32(-0.5)) * np.float32(2))
    # a run-time compiled lambda over two operands, one of them bf16 (the suite's softmax core: sum_k exp(x) * z)
    zb = oracle.f32_to_bf16(z)
    got = T.chain_reduce([xd, dev_bf16(zb, cuda)], "expf(p0) * f32(p1)", axis=1).cpu().numpy()
    want = (np.exp(x64) * oracle.bf16_to_f32(zb)).sum(1)
    assert (np.abs(got - want) <= 1e-5 * want + 1e-30).all()
    got = T.chain_reduce([xd, zd], "p0 * p1 + 0.25f", init=1.0, axis=1).cpu().numpy()
    want = (x64 * z + 0.25).sum(1) + 1.0
    assert (np.abs(got - want) <= 1e-5 * (np.abs(x64 * z) + 0.25).sum(1) + 1e-5).all()
    # sum, max and argmax in one pass: max and argmax bit-exact (ties on purpose: the lowest index wins), as with a
    # CTA per tile
    xt = np.round(x * 4).astype(np.float32) / 4
    got = T.reduce_outer(dev_f32(xt, cuda))
    assert np.array_equal(got["max"].cpu().numpy(), xt.max(1))
    assert np.array_equal(got["argmax"].cpu().numpy(), xt.argmax(1).astype(np.int32))
    assert (np.abs(got["sum"].cpu().numpy() - xt.astype(np.float64).sum(1)) <= 1e-5 * np.abs(xt).sum(1) + 1e-30).all()
    try:
        T.tune("reduce_outer", 0, 0, 0, 1)
        old = T.reduce_outer(dev_f32(xt, cuda))
    finally:
        T.tune("reduce_outer")
    assert torch.equal(old["max"], got["max"]) and torch.equal(old["argmax"], got["argmax"])
    only = T.reduce_outer(dev_f32(xt, cuda), want=("argmax",))
    assert torch.equal(only["argmax"], got["argmax"])


@pytest.mark.parametrize("nb,nk,nc", [(600, 300, 130), (40, 1000, 1023), (300, 500, 68), (2000, 70, 33), (50, 2000, 256)])
def test_middle_axis_warps_forced_on_other_shapes(oracle, cuda, nb, nk, nc):
    """The warp-per-tile kernels on shapes the library gives to a CTA per tile: same results."""
    rng = np.random.default_rng(nb + nk + nc)
    x = np.round(rng.uniform(-1, 1, (nb, nk, nc)) * 16).astype(np.float32) / 16
    xd = dev_f32(x, cuda)
    want = T.reduce_outer(xd)
    wsum = T.chain_reduce([xd], "p0 * p0", axis=1, init=0.25)
    try:
        T.tune("reduce_outer", 0, 1, 0, 0)
        T.tune("reduce_inner", 32, 0, 0, 0)
        got = T.reduce_outer(xd)
        gsum = T.chain_reduce([xd], "p0 * p0", axis=1, init=0.25)
    finally:
        T.tune("reduce_outer")
        T.tune("reduce_inner")
    assert torch.equal(got["max"], want["max"]) and torch.equal(got["argmax"], want["argmax"])
    assert np.array_equal(got["argmax"].cpu().numpy(), x.argmax(1).astype(np.int32))
    x64 = x.astype(np.float64)
    assert (np.abs(got["sum"].cpu().numpy() - x64.sum(1)) <= 1e-5 * np.abs(x64).sum(1) + 1e-30).all()
    ref = (x64 * x64).sum(1) + 0.25
    assert (np.abs(gsum.cpu().numpy() - ref) <= 1e-5 * ref).all() and (np.abs(wsum.cpu().numpy() - ref) <= 1e-5 * ref).all()


# ----------------------------------------------------------------------------
# column statistics of tall matrices: few column tiles, a long reduced axis -- the warps share the k axis too
# ----------------------------------------------------------------------------
@pytest.mark.parametrize("nb,nk,nc", [(1, 1 << 20, 8), (1, 262144, 128), (4, 131072, 64), (3, 100003, 16), (1, 70001, 512),
                                      (2, 40000, 1024), (1, 1 << 21, 4), (1, 1025, 32), (5, 30011, 260),
                                      (1, 700001, 3), (2, 100001, 7), (1, 150000, 20), (3, 50001, 30)])
def test_column_statistics_of_tall_matrices(oracle, cuda, nb, nk, nc):
    rng = np.random.default_rng(nb + nk + nc)
    x = rng.uniform(-1, 1, (nb, nk, nc)).astype(np.float32)
    xd = dev_f32(x, cuda)
    x64 = x.astype(np.float64)
    mag = np.abs(x64).sum(1)
    buf, out = guarded((nb, nc), torch.float32, cuda)
    n0 = T.launch_count()
    T.chain_reduce([xd], "p0", axis=1, out=out)
    assert T.launch_count() - n0 == 2          # the ranges, then their fold
    got = out.cpu().numpy()
    check_guards(buf, torch.float32)
    assert (np.abs(got - x64.sum(1)) <= 1e-6 * mag + 1e-30).all()
    # max with init and a piped map: bit-exact whatever the ranges
    got = T.chain_reduce([xd], "p0", combine_expr="fmaxf(p0, p1)", init=0.999, axis=1, post_expr="p0 * 2.0f").cpu().numpy()
    assert np.array_equal(got, np.maximum(x.max(1), np.float32(0.999)) * np.float32(2))
    # a run-time compiled lambda with a per-cell operand and an init (column variance around a given centre)
    c = rng.uniform(-0.1, 0.1, (nb, 1, nc)).astype(np.float32)
    got = T.chain_reduce([xd, dev_f32(c, cuda)], "(p0 - p1) * (p0 - p1)", init=0.5, axis=1).cpu().numpy()
    d = x64 - c.astype(np.float64)
    want = (d * d).sum(1) + 0.5
    assert (np.abs(got - want) <= 2e-6 * want).all()
    # sum, max and argmax in one pass; ties on purpose: the lowest index wins whichever range holds it
    xt = np.round(x * 8).astype(np.float32) / 8
    xtd = dev_f32(xt, cuda)
    n0 = T.launch_count()
    got = T.reduce_outer(xtd)
    assert T.launch_count() - n0 == 2
    assert np.array_equal(got["max"].cpu().numpy(), xt.max(1))
    assert np.array_equal(got["argmax"].cpu().numpy(), xt.argmax(1).astype(np.int32))
    assert (np.abs(got["sum"].cpu().numpy() - xt.astype(np.float64).sum(1)) <= 1e-6 * np.abs(xt).sum(1) + 1e-30).all()
    try:
        T.tune("reduce_outer", 1, 0, 0, 0)      # a CTA per column tile
        old = T.reduce_outer(xtd)
    finally:
        T.tune("reduce_outer")
    assert torch.equal(old["max"], got["max"]) and torch.equal(old["argmax"], got["argmax"])
    only = T.reduce_outer(xtd, want=("sum",))
    assert torch.equal(only["sum"], got["sum"])


# ----------------------------------------------------------------------------
# several problems of one shape in one launch
# ----------------------------------------------------------------------------
@pytest.mark.parametrize("nprob,rows,cols", [(16, 4096, 1024), (1, 5, 7), (3, 33, 130), (32, 17, 64), (2, 3, 9000), (5, 2, 4096)])
def test_batched_row_reductions_match_single_launches(oracle, cuda, nprob, rows, cols):
    from oracle import checks
    rng = np.random.default_rng(nprob * 7 + rows + cols)
    xs = [rng.uniform(-1, 1, (rows, cols)).astype(np.float32) for _ in range(nprob)]
    xd = [dev_f32(x, cuda) for x in xs]
    bufs = [guarded((rows,), torch.float32, cuda) for _ in range(nprob)]
    n0 = T.launch_count()
    T.chain_reduce_batched([[x] for x in xd], "(0.5f*p0 + 0.25f) * (0.5f*p0 + 0.25f)", outs=[o for _, o in bufs])
    assert T.launch_count() - n0 == 1
    for x, (buf, out) in zip(xs, bufs):
        check_guards(buf, torch.float32)
        assert checks.rowsum_close(out.cpu().numpy(), x)
    # two operands, a compiled lambda, max combiner with init, piped map
    zs = [rng.uniform(-1, 1, (rows, cols)).astype(np.float32) for _ in range(nprob)]
    zd = [dev_f32(z, cuda) for z in zs]
    got = T.chain_reduce_batched([[x, z] for x, z in zip(xd, zd)], "sinf(p0) * p1", post_expr="p0 * 0.5f + 1.0f")
    for x, z, g in zip(xs, zs, got):
        want = 0.5 * (np.sin(x.astype(np.float64)) * z).sum(1) + 1.0
        assert (np.abs(g.cpu().numpy() - want) <= 1e-5 * (0.5 * np.abs(np.sin(x.astype(np.float64)) * z).sum(1) + 1.0)).all()
    got = T.chain_reduce_batched([[x] for x in xd], "p0", combine_expr="fmaxf(p0, p1)", init=0.25)
    for x, g in zip(xs, got):
        assert np.array_equal(g.cpu().numpy(), np.maximum(x.max(1), np.float32(0.25)))
    # bit-identical to the single-problem entry on the same shapes (same kernels' fold order per row)
    single = T.chain_reduce([xd[0]], "p0").cpu().numpy()
    batched = T.chain_reduce_batched([[xd[0]]], "p0")[0].cpu().numpy()
    assert (np.abs(single - batched) <= 1e-5 * np.abs(xs[0]).sum(1)).all()


def test_batched_arguments_are_validated(cuda):
    x = torch.zeros((4, 8), device=cuda)
    with pytest.raises(ValueError):
        T.chain_reduce_batched([[x]] * 33, "p0")
    with pytest.raises(T.TcabError) as e:
        T.chain_reduce_batched([[x], [torch.zeros((4, 9), device=cuda)]], "p0")
    assert e.value.status == T._lib.ERR_SHAPE
    with pytest.raises(T.TcabError) as e:
        T.chain_reduce_batched([[x]], "p0", outs=[torch.zeros((5,), device=cuda)])
    assert e.value.status == T._lib.ERR_SHAPE


def test_small_problems_take_big_ctas_and_agree(oracle, cuda):
    # rows that fit the GPU at once are folded by 1024-thread CTAs (32 rows each); the tuning hook p2 = 3 keeps the
    # 128-thread shape: both must give the same sums (same warp-per-row fold)
    rng = np.random.default_rng(21)
    for rows, cols in [(4096, 1024), (64, 512), (9000, 260), (100, 4000)]:
        x = rng.uniform(-1, 1, (rows, cols)).astype(np.float32)
        xd = dev_f32(x, cuda)
        a = T.chain_reduce([xd], "p0 * p0").cpu().numpy()
        try:
            T.tune("reduce_inner", 0, 0, 3, 0)
            b = T.chain_reduce([xd], "p0 * p0").cpu().numpy()
        finally:
            T.tune("reduce_inner")
        assert np.array_equal(a, b)
        assert (np.abs(a - (x.astype(np.float64) ** 2).sum(1)) <= 1e-5 * (x.astype(np.float64) ** 2).sum(1)).all()

