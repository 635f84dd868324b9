"""The C-ABI library on a box without a GPU: it loads, exports exactly what
include/tcab.h declares, validates arguments like the reference's launcher
(named shape checks, internal/cg/cxx/launch.go:23-156) and refuses to compute
without a device. No compute call is made here."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols(header="tcab.h"):
    text = open(os.path.join(ROOT, "include", header)).read()
    return sorted(set(re.findall(r"^TCAB_API[^;]*?\b(tcab_\w+)\s*\(", text, flags=re.M | re.S)))


def test_every_declared_symbol_is_exported(tcab_lib):
    from tcacomp_b200 import _lib
    names = declared_symbols()
    assert len(names) >= 10
    for n in names:
        assert hasattr(tcab_lib, n), f"{n} declared in include/tcab.h but not exported"
    assert sorted(s[0] for s in _lib.SYMBOLS) == names, "ctypes table and header disagree"
    tuning = declared_symbols("tcab_tuning.h")
    for n in tuning:
        assert hasattr(tcab_lib, n), f"{n} declared in include/tcab_tuning.h but not exported"
    assert sorted(s[0] for s in _lib.TUNING_SYMBOLS) == tuning, "ctypes table and tuning header disagree"
    assert "tcab_tuning.h" not in open(os.path.join(ROOT, "include", "tcab.h")).read()
    assert tcab_lib.tcab_abi_version() == 1


def _tensor(shape, dtype=0, data=0x1000):
    from tcacomp_b200 import _lib
    t = _lib.Tensor()
    t.data, t.dtype, t.rank = data, dtype, len(shape)
    for i, d in enumerate(shape):
        t.dims[i] = d
    return t


def _err(lib):
    return lib.tcab_last_error().decode()


def test_shape_and_dtype_validation_precede_any_launch(tcab_lib):
    from tcacomp_b200 import _lib
    L = tcab_lib
    x, y = _tensor((4, 8)), _tensor((4, 9))
    assert L.tcab_softmax_rows(C.byref(x), C.byref(y), None) == _lib.ERR_SHAPE
    assert "shape of x" in _err(L)
    assert L.tcab_softmax_rows(None, C.byref(y), None) == _lib.ERR_INVALID_ARG
    xb = _tensor((4, 8), dtype=_lib.BF16)
    assert L.tcab_softmax_rows(C.byref(xb), C.byref(xb), None) == _lib.ERR_DTYPE
    bad_rank = _tensor((4, 8))
    bad_rank.rank = 7
    assert L.tcab_softmax_rows(C.byref(bad_rank), C.byref(bad_rank), None) == _lib.ERR_INVALID_ARG
    null = _tensor((4, 8), data=0)
    assert L.tcab_softmax_rows(C.byref(null), C.byref(null), None) == _lib.ERR_INVALID_ARG
    odd = _tensor((4, 8), data=0x1002)
    assert L.tcab_softmax_rows(C.byref(odd), C.byref(odd), None) == _lib.ERR_ALIGNMENT

    g = _tensor((7,), dtype=_lib.BF16)
    xb = _tensor((4, 8), dtype=_lib.BF16)
    assert L.tcab_layernorm_rows(C.byref(xb), C.byref(g), C.byref(g), 1e-5, C.byref(xb), None) == _lib.ERR_SHAPE
    assert "gamma" in _err(L)

    t = _tensor((2, 3, 4))
    s_bad = _tensor((2, 5))
    assert L.tcab_reduce_outer(C.byref(t), C.byref(s_bad), None, None, None) == _lib.ERR_SHAPE
    assert L.tcab_reduce_outer(C.byref(t), None, None, None, None) == _lib.ERR_INVALID_ARG
    am_f32 = _tensor((2, 4))
    assert L.tcab_reduce_outer(C.byref(t), None, None, C.byref(am_f32), None) == _lib.ERR_DTYPE

    a, b, c = _tensor((16, 32), _lib.BF16), _tensor((24, 8), _lib.BF16), _tensor((16, 8), _lib.BF16)
    assert L.tcab_gemm_bias_act(C.byref(a), C.byref(b), None, 1, C.byref(c), None) == _lib.ERR_SHAPE
    assert "dim k" in _err(L)
    b = _tensor((32, 12), _lib.BF16)
    c = _tensor((16, 12), _lib.BF16)
    assert L.tcab_gemm_bias_act(C.byref(a), C.byref(b), None, 1, C.byref(c), None) == _lib.ERR_ALIGNMENT

    big = _tensor((70000, 70000))
    assert L.tcab_softmax_rows(C.byref(big), C.byref(big), None) == _lib.ERR_TOO_LARGE


def _chain(map_expr, combine="(p0 + p1)", post=None, caps=()):
    from tcacomp_b200 import _lib
    ch = _lib.Chain()
    ch.map_expr, ch.combine_expr = map_expr.encode(), combine.encode()
    ch.post_expr = post.encode() if post else None
    ch.init, ch.n_captures = 0.0, len(caps)
    for i, v in enumerate(caps):
        ch.captures[i] = v
    return ch


def test_chain_lambdas_are_validated_on_the_host(tcab_lib):
    from tcacomp_b200 import _lib
    L = tcab_lib
    x, out = _tensor((4, 8)), _tensor((4,))
    arr = (_lib.Tensor * 1)(x)

    def call(ch, n=1, axis=1, o=out):
        return L.tcab_chain_reduce(C.byref(ch), arr, n, axis, C.byref(o), None)

    assert call(_chain("system(p0)")) == _lib.ERR_INVALID_ARG and "unknown identifier" in _err(L)
    assert call(_chain("p0 +")) == _lib.ERR_INVALID_ARG
    assert call(_chain("p0; p0")) == _lib.ERR_INVALID_ARG
    assert call(_chain("p1")) == _lib.ERR_INVALID_ARG and "out of range" in _err(L)
    assert call(_chain("c0 * p0")) == _lib.ERR_INVALID_ARG  # capture not supplied
    assert call(_chain("p0", combine="(p0 * p1)")) == _lib.ERR_UNSUPPORTED
    # a lambda without an ahead-of-time kernel is compiled at run time, which needs the device:
    # on a box without one the call gets as far as the device check and no further
    assert call(_chain("sinf(cosf(p0))")) == _lib.ERR_CUDA or _has_gpu()
    assert call(_chain("p0"), o=_tensor((5,))) == _lib.ERR_SHAPE
    assert call(_chain("p0"), axis=2) == _lib.ERR_INVALID_ARG
    # a well-formed chain with a compiled kernel gets as far as the device check
    assert call(_chain("(0.5f*p0 + 0.25f) * (0.5f*p0 + 0.25f)")) == _lib.ERR_CUDA or _has_gpu()
    assert call(_chain("c0*p0 + c1", caps=(1.0,))) == _lib.ERR_INVALID_ARG


def _has_gpu():
    import torch
    return torch.cuda.is_available()


def test_compute_without_a_device_fails_loudly(tcab_lib):
    if _has_gpu():
        pytest.skip("a CUDA device is present")
    from tcacomp_b200 import _lib
    x = _tensor((4, 8))
    assert tcab_lib.tcab_softmax_rows(C.byref(x), C.byref(x), None) == _lib.ERR_CUDA
    assert "no CPU path" in _err(tcab_lib)


def test_python_host_rejects_cpu_tensors():
    import torch
    import tcacomp_b200 as T
    with pytest.raises(ValueError, match="no CPU path"):
        T.softmax_rows(torch.zeros(4, 4))


def test_tune_rejects_unknown_family(tcab_lib):
    from tcacomp_b200 import _lib
    assert tcab_lib.tcab_tune(b"nope", 1, 1, 1, 0) == _lib.ERR_INVALID_ARG
    assert tcab_lib.tcab_tune(b"softmax", 0, 0, 0, 0) == _lib.OK


def test_python_views_refuse_what_32_bit_extents_cannot_hold():
    # ctypes truncates a value >= 2^32 stored into a c_uint32 field without an error; the Python view must not
    import torch
    from tcacomp_b200 import ops
    with pytest.raises(ValueError, match="32-bit"):
        ops._view(torch.empty((2**32,), device="meta"), "x")
    with pytest.raises(ValueError, match="32-bit"):
        ops._view(torch.empty((2**16, 2**16), device="meta"), "x")
    with pytest.raises(ValueError, match="CUDA device"):
        ops._view(torch.empty((4, 4)), "x")


def _bchain(map_expr, combine=b"(p0 + p1)", post=None):
    from tcacomp_b200 import _lib
    ch = _lib.Chain()
    ch.map_expr, ch.combine_expr, ch.post_expr = map_expr, combine, post
    return ch


def test_prepare_and_release_validate_without_a_device(tcab_lib):
    from tcacomp_b200 import _lib
    L = tcab_lib
    ch = _bchain(b"sinf(p0) * p1")
    assert L.tcab_chain_prepare(C.byref(ch), None, 2, 7, 0) == _lib.ERR_INVALID_ARG          # unknown use
    assert L.tcab_chain_prepare(C.byref(ch), None, 3, _lib.USE_CONTRACT, 0) == _lib.ERR_INVALID_ARG  # contractions take two
    bad = _bchain(b"sinf(p0) * q1")
    assert L.tcab_chain_prepare(C.byref(bad), None, 2, _lib.USE_REDUCE, 0) == _lib.ERR_INVALID_ARG   # the lambda is validated first
    import torch
    if not torch.cuda.is_available():
        assert L.tcab_chain_prepare(C.byref(ch), None, 2, _lib.USE_REDUCE, 0) == _lib.ERR_CUDA      # compiling needs the device
        assert L.tcab_release_stream(None) == _lib.ERR_CUDA
    assert L.tcab_release_all() == _lib.OK                                               # nothing held: nothing to free


F, B, I, U = 0, 1, 2, 3

# (lambda, operand types, use, output type): the reference's typed vocabulary (pkg/expr.go:137-176, 185-203, 271;
# operator spellings internal/cg/cxx/naming.go:126-183), every form once. Each is validated, printed as a typed
# functor and compiled for sm_100a by the run-time compiler -- no GPU needed for that.
TYPED_OK = [
    (b"p0 > 0.0f ? p0 : 0.0f", [F], "map", F),                                  # Select(Gt(v, 0), v, 0): relu
    (b"(p0 >= p1 && p0 != 1.0f) || !(p1 <= 2.0f) ? p0 - p1 : -p0 / p1", [F, F], "map", F),
    (b"p0 == p1 ? 1 : 0", [F, F], "map", I),
    (b"bf16(fmaxf(f32(p0) * f32(p1) + 1.0f, 0.0f))", [B, B], "map", B),         # Cast bf16 -> f32 -> bf16
    (b"static_cast<float>(p0)", [B], "map", F),
    (b"(p0 & 255) << 3 | p1 >> 1 ^ ~p0 % 7", [I, I], "map", I),                # Mod BitAnd BitOr BitXor Shl Shr BitsNot
    (b"umin(p0, 7u) + umax(p1, p0) * 3u - (p0 >> 1u)", [U, U], "map", U),
    (b"i32(p0) + i32(f32(p1))", [F, B], "map", I),
    (b"u32(p0) < 5u ? f32(p0) : fabsf(f32(p0))", [I], "map", F),
    (b"f32(p0) * p1", [B, F], "reduce", F),                                     # bf16 operand widened inside a reduction
    (b"(p0 % 3 == 0 ? 2.0f : 0.5f) * p1", [I, F], "reduce", F),
    (b"sinf(p0) * f32(p1)", [F, B], "reduce_batched", F),                       # several problems in one launch
    (b"f32(p0) * f32(p1)", [B, B], "contract", F),                              # bf16 operands of a contraction
]
TYPED_BAD = [
    (b"p0 * 2", [F], "map", F, b"operand types differ"),                         # no implicit promotion
    (b"p0 + p1", [F, I], "map", F, b"operand types differ"),
    (b"p0 * p1", [B, B], "map", B, b"convert bf16 to f32 first"),                # bf16 is a storage type
    (b"p0 % p1", [F, F], "map", F, b"same integer type"),
    (b"p0 && p1", [F, F], "map", F, b"must be bool"),
    (b"p0 ? p1 : p0", [F, F], "map", F, b"condition must be bool"),
    (b"p0 < p1 ? 1 : 2u", [F, F], "map", I, b"identical types"),
    (b"f32(p0)", [F], "map", F, b"redundant cast"),
    (b"f32(p0 < p1)", [F, F], "map", F, b"bool cannot be converted"),
    (b"~p0", [F], "map", F, b"integer type"),
    (b"p0", [F], "map", B, b"convert explicitly"),                               # the store never converts
    (b"i32(p0)", [F], "reduce", F, b"folds f32 values"),
    (b"expf(p0)", [I], "map", F, b"must be f32"),
    (b"umin(p0, p1)", [I, I], "map", I, b"must be u32"),
    (b"4294967296u", [F], "map", U, b"out of range"),
]


def _use(name):
    from tcacomp_b200 import _lib
    return {"reduce": _lib.USE_REDUCE, "contract": _lib.USE_CONTRACT, "map": _lib.USE_MAP,
            "reduce_batched": _lib.USE_REDUCE_BATCHED}[name]


@pytest.mark.parametrize("expr,types,use,out", TYPED_OK)
def test_typed_lambdas_compile_for_sm100(tcab_lib, expr, types, use, out):
    from tcacomp_b200 import _lib
    ch = _bchain(expr)
    arr = (C.c_int32 * len(types))(*types)
    rc = tcab_lib.tcab_compile_check(C.byref(ch), arr, len(types), _use(use), out, 0, 0, 0)
    assert rc == _lib.OK, _err(tcab_lib)


@pytest.mark.parametrize("expr,types,use,out,why", TYPED_BAD)
def test_ill_typed_lambdas_are_refused_before_any_compiler(tcab_lib, expr, types, use, out, why):
    from tcacomp_b200 import _lib
    ch = _bchain(expr)
    arr = (C.c_int32 * len(types))(*types)
    rc = tcab_lib.tcab_compile_check(C.byref(ch), arr, len(types), _use(use), out, 0, 0, 0)
    assert rc in (_lib.ERR_INVALID_ARG, _lib.ERR_DTYPE), (rc, _err(tcab_lib))
    assert why in tcab_lib.tcab_last_error(), _err(tcab_lib)


def test_partition_rule_and_pipeline_validation_without_a_device(tcab_lib):
    from tcacomp_b200 import _lib, shard
    L = tcab_lib
    lo, hi = C.c_uint64(), C.c_uint64()
    for n in (0, 1, 7, 1003, 65536):
        for world in (1, 2, 3, 8):
            covered = 0
            for r in range(world):
                assert L.tcab_shard_block(n, world, r, C.byref(lo), C.byref(hi)) == _lib.OK
                assert (lo.value, hi.value) == shard.block(n, world, r) and lo.value == covered
                covered = hi.value
            assert covered == n
    assert L.tcab_shard_block(10, 2, 2, C.byref(lo), C.byref(hi)) == _lib.ERR_INVALID_ARG
    d = _lib.PipelineDesc()
    d.op, d.device, d.chunk_units, d.in_dtype, d.n_streamed, d.unit_rank = _lib.OP_SOFTMAX_ROWS, -1, 16, _lib.F32, 1, 1
    d.unit_dims[0] = 512
    h = C.c_void_p()
    d.chunk_units = 0
    assert L.tcab_pipeline_create(C.byref(d), C.byref(h)) == _lib.ERR_INVALID_ARG and not h.value
    d.chunk_units, d.depth = 16, 9
    assert L.tcab_pipeline_create(C.byref(d), C.byref(h)) == _lib.ERR_INVALID_ARG
    d.depth, d.in_dtype = 0, _lib.BF16
    assert L.tcab_pipeline_create(C.byref(d), C.byref(h)) == _lib.ERR_DTYPE          # softmax rows are f32
    d.in_dtype, d.op = _lib.F32, _lib.OP_LAYERNORM_ROWS
    assert L.tcab_pipeline_create(C.byref(d), C.byref(h)) == _lib.ERR_INVALID_ARG    # gamma / beta missing
    import torch
    if not torch.cuda.is_available():
        d.op = _lib.OP_SOFTMAX_ROWS
        assert L.tcab_pipeline_create(C.byref(d), C.byref(h)) == _lib.ERR_CUDA and not h.value   # no CPU path
    assert L.tcab_pipeline_destroy(None) == _lib.OK and L.tcab_multi_destroy(None) == _lib.OK


@pytest.mark.parametrize("expr,types,use,out,rb,cb,cells", [
    (b"expf(p0 - p1)", [F, F], "reduce", F, 0b10, 0, 0),              # sum_j exp(x[i][j] - m[i]): reads a row maximum
    (b"expf(p0 - p1) / p2", [F, F, F], "map", F, 0b110, 0, 0),       # the normalising map of a softmax
    (b"bf16((f32(p0) - p1) * p2 * f32(p3) + f32(p4))", [B, F, F, B, B], "map", B, 0b00110, 0b11000, 0),   # layer-norm's last map
    (b"fmaxf(p0 + p1, 0.0f)", [F, F], "map", F, 0, 0b10, 0),         # bias[n] and ReLU
    (b"expf(p0 - p1) * f32(p2)", [F, F, B], "reduce", F, 0, 0, 0b010),   # middle-axis: sum_k exp(x[i][k][j] - m[i][j]) * z
])
def test_lambdas_over_operands_that_bind_a_subset_of_the_axes_compile(tcab_lib, expr, types, use, out, rb, cb, cells):
    from tcacomp_b200 import _lib
    ch = _bchain(expr)
    arr = (C.c_int32 * len(types))(*types)
    assert tcab_lib.tcab_compile_check(C.byref(ch), arr, len(types), _use(use), out, rb, cb, cells) == _lib.OK, _err(tcab_lib)


def test_register_row_shapes(tcab_lib):
    """The shape a register-row kernel gets: every row is covered, rows of 3 * 2^k and 5 * 2^k vectors (hidden sizes
    768, 1280, 1536, 2560, 3072, 5120 ...) fit exactly with every slot used, powers of two keep four slots."""
    def shape(op, eb, nvec):
        t, v = C.c_uint32(), C.c_uint32()
        assert tcab_lib.tcab_plan_row_shape(op, eb, nvec, C.byref(t), C.byref(v)) == 0
        return t.value, v.value
    for op, eb in ((0, 4), (1, 4), (1, 2)):
        for nvec in list(range(1, 600)) + [640, 768, 1000, 1024, 1280, 1536, 2048, 2560, 3000, 4096]:
            t, v = shape(op, eb, nvec)
            assert t * v >= nvec and t >= 1 and (t & (t - 1)) == 0, (op, eb, nvec, t, v)
            assert -(-nvec // t) > v - (2 if v <= 4 else v // 2), (op, eb, nvec, t, v)     # no shape mostly empty
    # bf16 layer-norm: 640, 768, 1280, 1536, 2560, 3072, 5120, 6144, 10240, 12288 columns
    assert [shape(1, 2, n) for n in (80, 96, 160, 192, 320, 384, 640, 768, 1280, 1536)] == \
        [(16, 5), (32, 3), (32, 5), (64, 3), (64, 5), (128, 3), (128, 5), (256, 3), (256, 5), (512, 3)]
    # fp32 layer-norm and softmax: three slots everywhere, five only with at most 32 threads per row
    assert shape(1, 4, 160) == (32, 5) and shape(1, 4, 320) != (64, 5) and shape(1, 4, 1280) != (256, 5)
    assert shape(1, 4, 192) == (64, 3) and shape(1, 4, 1536) == (512, 3) and shape(0, 4, 384) == (128, 3)
    # powers of two: four slots (bf16 C3: 8192 columns = 1024 vectors; fp32 C2: 4096 columns = 1024 vectors)
    assert shape(1, 2, 1024) == (256, 4) and shape(0, 4, 1024) == (256, 4) and shape(1, 4, 256) == (64, 4)
    assert tcab_lib.tcab_plan_row_shape(0, 2, 64, C.byref(C.c_uint32()), C.byref(C.c_uint32())) != 0    # softmax is fp32
    assert tcab_lib.tcab_plan_row_shape(2, 4, 64, C.byref(C.c_uint32()), C.byref(C.c_uint32())) != 0


def test_outer_flat_ranges(tcab_lib):
    """Few narrow column tiles and a long reduced axis: CTAs of the warp-per-tile kernels cut k into ranges that cover it,
    none empty, within the scratch for the partial cells (one per range); many tiles, wide tiles or a short axis are
    never cut."""
    def plan(nb, nk, nc, sms=148, cap=262144):
        g, r, kl = C.c_uint32(), C.c_uint32(), C.c_uint32()
        assert tcab_lib.tcab_plan_outer_flat_ranges(nb, nk, nc, sms, cap, C.byref(g), C.byref(r), C.byref(kl)) == 0
        return g.value, r.value, kl.value
    for nb, nk, nc in [(1, 1 << 25, 4), (1, 1 << 23, 16), (1, 1 << 20, 64), (4, 524288, 64), (700, 5000, 32),
                       (3, 100003, 8), (1, 1025, 4), (2, 5000, 16), (1000, 1 << 16, 64)]:
        g, r, kl = plan(nb, nk, nc)
        assert g == nc // 4 and r >= 1 and kl >= 1
        assert (r - 1) * kl < nk <= r * kl                      # the ranges cover k and the last one is not empty
        assert r == 1 or nb * nc * r <= 262144                  # partial cells fit the scratch
        assert r == 1 or kl >= (32 // g) * 8 * 16               # at least 16 steps per warp of a range
    assert plan(1, 1 << 25, 4)[1] == 1184 and plan(1, 1 << 20, 64)[1] == 1184  # eight CTAs per SM
    assert plan(700, 5000, 8)[1] == 2 and plan(1000, 1 << 16, 16)[1] == 2      # rounded up to fill the GPU
    assert plan(700, 5000, 32)[1] == 2 and plan(1000, 1 << 16, 64)[1] == 2
    assert plan(1000, 1 << 16, 64, cap=100000)[1] == 1          # 64000 cells: two ranges would overrun this scratch
    assert plan(1, 1025, 4)[1] == 1                             # too short for two ranges
    assert plan(100000, 256, 16)[1] == 1 and plan(2000, 1 << 16, 32)[1] == 1   # many tiles: one warp per tile
    assert plan(1, 1 << 20, 128) == (0, 1, 1 << 20) and plan(1, 1 << 20, 512)[0] == 0   # wide tiles: a CTA per tile
    assert plan(1, 1 << 20, 16, cap=128)[1] == 8                # a small scratch bounds the ranges


def test_row_kernel_shape_rules(tcab_lib):
    """The launchers' choices that are pure arithmetic: which middle-axis shapes a warp per (b, column tile) takes, how
    many CTAs stream a long row, how many warps the thread-per-row kernel gets."""
    def plan(rows=0, nk=1, nc=4, sms=148, nvec=1, per_step=1024, three=1, n_in=1):
        g, cs, w = C.c_uint32(), C.c_uint32(), C.c_uint32()
        assert tcab_lib.tcab_plan_row_kernels(rows, nk, nc, sms, nvec, per_step, three, n_in, C.byref(g), C.byref(cs), C.byref(w)) == 0
        return g.value, cs.value, w.value
    # narrow rows: the whole row is one tile of nc / 4 column groups
    assert [plan(rows=100000, nk=256, nc=c)[0] for c in (4, 8, 16, 32)] == [1, 2, 4, 8]
    assert plan(rows=100000, nk=256, nc=64)[0] == 16 and plan(rows=1000, nk=256, nc=64)[0] == 0   # 64 columns: only with many warps
    assert plan(rows=100000, nk=256, nc=12)[0] == 3 and plan(rows=100000, nk=256, nc=48)[0] == 12  # any number of groups
    assert plan(rows=100000, nk=256, nc=96)[0] == 0 and plan(rows=100000, nk=16, nc=96)[0] == 24   # 65 ... 127 columns: short axes
    # rows that are not whole vectors: groups of one column, tiles of 32 columns
    assert [plan(rows=100000, nk=256, nc=c)[0] for c in (1, 3, 6, 7, 31)] == [1, 3, 6, 7, 31]
    assert plan(rows=100000, nk=256, nc=33)[0] == 32 and plan(rows=100000, nk=8, nc=2050)[0] == 32
    assert plan(rows=2, nk=1 << 20, nc=33)[0] == 0 and plan(rows=2, nk=1 << 20, nc=15)[0] == 15   # few long columns
    # short reduced axes with wide rows: 32 groups of a 128-column tile; long axes keep a CTA per tile
    assert plan(rows=65536, nk=4, nc=1024)[0] == 32 and plan(rows=65536, nk=64, nc=1024)[0] == 0
    # a handful of long columns: the warps share the k axis as well (test_outer_flat_ranges)
    assert plan(rows=8, nk=1 << 20, nc=8)[0] == 2 and plan(rows=8, nk=4096, nc=8)[0] == 2
    assert plan(rows=1, nk=1 << 20, nc=512)[0] == 0 and plan(rows=1, nk=1 << 20, nc=96)[0] == 0
    # streaming clusters: four steps with the smallest cluster, three full steps where a larger one gives them
    assert plan(nvec=6144)[1] == 2 and plan(nvec=8192)[1] == 4 and plan(nvec=12564)[1] == 4 and plan(nvec=32768)[1] == 8
    assert plan(nvec=8192, three=0)[1] == 2 and plan(nvec=100)[1] == 2 and plan(nvec=10**6, per_step=4096)[1] == 8
    # thread-per-row kernel: 8 warps while 48 KiB hold them, fewer with more operands, none when one warp does not fit
    assert plan(nvec=16, n_in=1)[2] == 5 and plan(nvec=4, n_in=1)[2] == 8 and plan(nvec=16, n_in=6)[2] == 0
    assert plan(nvec=16, n_in=2)[2] == 2 and plan(nvec=16, n_in=3)[2] == 1
