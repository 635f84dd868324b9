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


def test_prepare_and_release_validate_without_a_device(tcab_lib):
    from tcacomp_b200 import _lib
    L = tcab_lib
    ch = _lib.Chain()
    ch.map_expr, ch.combine_expr = b"sinf(p0) * p1", b"(p0 + p1)"
    assert L.tcab_chain_prepare(C.byref(ch), 2, 7) == _lib.ERR_INVALID_ARG          # unknown use
    assert L.tcab_chain_prepare(C.byref(ch), 3, _lib.USE_CONTRACT) == _lib.ERR_INVALID_ARG  # contractions take two
    ch.map_expr = b"sinf(p0) * q1"
    assert L.tcab_chain_prepare(C.byref(ch), 2, _lib.USE_REDUCE) == _lib.ERR_INVALID_ARG    # the lambda is validated first
    import torch
    if not torch.cuda.is_available():
        ch.map_expr = b"sinf(p0) * p1"
        assert L.tcab_chain_prepare(C.byref(ch), 2, _lib.USE_REDUCE) == _lib.ERR_CUDA      # compiling needs the device
        assert L.tcab_release_stream(None) == _lib.ERR_CUDA
    assert L.tcab_release_all() == _lib.OK                                               # nothing held: nothing to free
