"""The .tca text frontend through its C ABI (include/tcab_host.h, tcacomp_b200/tca.py).

CPU half: libtcab_host.so exports what the header declares; modules parse, classify and report errors with
positions, the way the reference's parser and semacheck tests do (internal/syntax/parser/parser_test.go,
internal/syntax/semacheck/*_test.go). GPU half: kernels written as text run on the device and are compared
with the oracle, the way internal/e2e/frontend_test.go takes matmul_scale from text to numbers."""
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

AFFINE_ROWSUM = '''
// C1-shaped: y[i] = sum_j (s * x[i][j] + t)^2
@name(cxx="AffineSqRowsum")
kernel affine_sq_rowsum(x: tensor<dtype=f32, shape=[R, C]>, s: f32, t: f32) -> tensor<dtype=f32, shape=[R]> {
  dimvar (i, j);
  let y = map on(x[i][j]) [s, t] (v: f32) -> f32: (s * v + t) * (s * v + t)
        | reduce(init = 0.0f) on(acc: f32, %0: f32) as (i) -> f32: acc + %0;
  return y;
}
'''

SCALED_MATMUL = '''
@name(cxx="ScaledMatmul")
kernel scaled_matmul(lhs: tensor<dtype=f32, shape=[M, N]>, rhs: tensor<dtype=f32, shape=[N, K]>, scale: f32)
    -> tensor<dtype=f32, shape=[M, K]> {
  dimvar (m, k, n);
  let out = map on(lhs[m][n], rhs[n][k]) (l: f32, r: f32) -> f32: l * r
          | reduce(init = 0.0f) on(acc: f32, %0: f32) as (m, k) -> f32: acc + %0
          | map on() [scale] (v: f32) -> f32: v * scale;
  return out;
}
'''

BF16_GEMM = '''
@name(cxx="GemmBiasRelu")
kernel gemm_bias_relu(a: tensor<dtype=bf16, shape=[M, K]>, b: tensor<dtype=bf16, shape=[K, N]>,
                      bias: tensor<dtype=f32, shape=[N]>) -> tensor<dtype=bf16, shape=[M, N]> {
  dimvar (m, n, k);
  let c = map on(a[m][k], b[k][n]) (l: bf16, r: bf16) -> f32: f32(l) * f32(r)
        | reduce(init = 0.0f) on(acc: f32, %0: f32) as (m, n) -> f32: acc + %0
        | map on(bias[n]) (v: f32, bb: f32) -> bf16: bf16(fmaxf(v + bb, 0.0f));
  return c;
}
'''


def test_host_library_exports_what_the_header_declares():
    from tcacomp_b200 import tca
    text = open(os.path.join(ROOT, "include", "tcab_host.h")).read()
    names = sorted(set(re.findall(r"^TCAB_API[^;]*?\b(tcab_\w+)\s*\(", text, flags=re.M | re.S)))
    lib = tca.load()
    assert len(names) >= 11
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/tcab_host.h but not exported"
    assert sorted(s[0] for s in tca.SYMBOLS) == names


def test_modules_parse_and_classify():
    from tcacomp_b200 import tca
    m = tca.Module(AFFINE_ROWSUM + SCALED_MATMUL + BF16_GEMM)
    assert m.names() == ["AffineSqRowsum", "ScaledMatmul", "GemmBiasRelu"]
    assert m.kernels["AffineSqRowsum"] == {"output": "y", "class": "chain_reduce"}
    assert m.kernels["ScaledMatmul"] == {"output": "out", "class": "chain_contract"}
    assert m.kernels["GemmBiasRelu"] == {"output": "c", "class": "gemm_bias_act"}


@pytest.mark.parametrize("text,status,needle", [
    ("kernel k(x: tensor<dtype=f32, shape=[R, 4]>) -> f32 { }", 1, "1:41: a constant extent is an unsigned literal"),
    ("kernel k(x: tensor<dtype=f32, shape=[R]>) -> tensor<dtype=f32, shape=[R]> {\n  dimvar i;\n"
     "  let o = map on(x[i]) (v: f32): v | map on() (w: f32): w;\n  return o; }", 1, "a second map needs a reduction before it"),
    ('@include "other.tca";', 1, 'missing include file "other.tca"'),
    ('@include "/etc/other.tca";', 1, "must be relative to the including file"),
    ('@include "../other.tca";', 1, "escapes the including file's directory"),
    (AFFINE_ROWSUM.replace("[s, t]", "[s]"), 1, "'t' is used but not captured"),
    (AFFINE_ROWSUM.replace("x[i][j]", "x[i]"), 1, "has rank 2, subscripted with 1"),
    (AFFINE_ROWSUM.replace("acc + %0", "acc < %0 ? acc : 1"), 1, "select: branches must have identical types"),
    (AFFINE_ROWSUM.replace("(s * v + t) * (s * v + t)", "v * 2"), 1, "operand types differ (f32 vs i32)"),
    (AFFINE_ROWSUM.replace("(s * v + t) * (s * v + t)", "v > 0.0f"), 1, "homogeneous reducer"),
    (AFFINE_ROWSUM.replace("return y;", "return z;"), 1, "'return' must name a let-bound tensor"),
    (AFFINE_ROWSUM.replace("return y;", "let y = map on(x[i][j]) (v: f32): v; return y;"), 1, "already bound"),
])
def test_diagnostics(text, status, needle):
    from tcacomp_b200 import TcabError, tca
    with pytest.raises(TcabError) as e:
        tca.Module(text)
    assert e.value.status == status, e.value.message
    assert needle in e.value.message
    assert re.match(r"\d+:\d+: ", e.value.message)


SOFTMAX_BY_STATEMENTS = '''
// Row softmax written statement by statement: the two reductions store into locals (pkg/builder.go:224,
// pkg/local_test.go:17-68), the last statement is the rank-preserving map.
@name(cxx="SoftmaxRows")
kernel softmax_rows(x: tensor<dtype=f32, shape=[R, C]>) -> tensor<dtype=f32, shape=[R, C]> {
  dimvar (i, j);
  let m = map on(x[i][j]) (v: f32) -> f32: v
        | reduce(init = -inf_f32) on(acc: f32, %0: f32) as (i) -> f32: fmaxf(acc, %0);
  let s = map on(x[i][j], m[i]) (v: f32, mx: f32) -> f32: expf(v - mx)
        | reduce(init = 0.0f) on(acc: f32, %0: f32) as (i) -> f32: acc + %0;
  let y = map on(x[i][j], m[i], s[i]) (v: f32, mx: f32, sum: f32) -> f32: expf(v - mx) / sum;
  return y;
}
'''

LAYERNORM_BY_STATEMENTS = '''
@name(cxx="LayernormRows")
kernel layernorm_rows(x: tensor<dtype=bf16, shape=[R, C]>, gamma: tensor<dtype=bf16, shape=[C]>,
                      beta: tensor<dtype=bf16, shape=[C]>, inv_n: f32, eps: f32) -> tensor<dtype=bf16, shape=[R, C]> {
  dimvar (i, j);
  let mean = map on(x[i][j]) (v: bf16) -> f32: f32(v)
           | reduce(init = 0.0f) on(acc: f32, %0: f32) as (i) -> f32: acc + %0
           | map on() [inv_n] (t: f32) -> f32: t * inv_n;
  let var = map on(x[i][j], mean[i]) (v: bf16, mu: f32) -> f32: (f32(v) - mu) * (f32(v) - mu)
          | reduce(init = 0.0f) on(acc: f32, %0: f32) as (i) -> f32: acc + %0
          | map on() [inv_n] (t: f32) -> f32: t * inv_n;
  let y = map on(x[i][j], mean[i], var[i], gamma[j], beta[j]) [eps]
            (v: bf16, mu: f32, s2: f32, g: bf16, b: bf16) -> bf16:
              bf16((f32(v) - mu) * rsqrtf(s2 + eps) * f32(g) + f32(b));
  return y;
}
'''

MASKED_NORMALISER_MIDDLE_AXIS = '''
// The reference's suite softmax reduces over the MIDDLE axis with a mask operand and without the row maximum
// (testing/kernels/fusion/softmax.tca:1-21 records why). With locals the stable form is two statements; the second
// reads the first one's result by the two axes that remain: one value per output cell. (A local of rank 2 needs
// static extents, as in the reference's builder.)
@name(cxx="MaskedNormaliser")
kernel masked_normaliser(x: tensor<dtype=f32, shape=[7u, 50u, 132u]>, z: tensor<dtype=f32, shape=[7u, 50u, 132u]>)
    -> tensor<dtype=f32, shape=[7u, 132u]> {
  dimvar (i, k, j);
  let m = map on(x[i][k][j]) (v: f32) -> f32: v
        | reduce(init = -inf_f32) on(acc: f32, %0: f32) as (i, j) -> f32: fmaxf(acc, %0);
  let out = map on(x[i][k][j], m[i][j], z[i][k][j]) (v: f32, mx: f32, w: f32) -> f32: expf(v - mx) * w
          | reduce(init = 0.0f) on(acc: f32, %0: f32) as (i, j) -> f32: acc + %0;
  return out;
}
'''

TYPED_KERNELS = '''
@name(cxx="ReluSelect")
kernel relu_select(x: tensor<dtype=f32, shape=[R, C]>) -> tensor<dtype=f32, shape=[R, C]> {
  dimvar (i, j);
  let y = map on(x[i][j]) (v: f32) -> f32: v > 0.0f ? v : 0.0f;     // Select(Gt(v, 0), v, 0)
  return y;
}
@name(cxx="CountMultiples")
kernel count_multiples(k: tensor<dtype=i32, shape=[R, C]>, w: tensor<dtype=f32, shape=[R, C]>) -> tensor<dtype=f32, shape=[R]> {
  dimvar (i, j);
  let n = map on(k[i][j], w[i][j]) (a: i32, b: f32) -> f32: ((a % 3 == 0 && a != 9) || (a & 1) == 1 ? 1.0f : 0.0f) * b
        | reduce(init = 0.0f) on(acc: f32, %0: f32) as (i) -> f32: acc + %0;
  return n;
}
@name(cxx="BiasRelu")
kernel bias_relu(x: tensor<dtype=f32, shape=[R, C]>, bias: tensor<dtype=f32, shape=[C]>) -> tensor<dtype=bf16, shape=[R, C]> {
  dimvar (i, j);
  let y = map on(x[i][j], bias[j]) (v: f32, b: f32) -> bf16: bf16(fmaxf(v + b, 0.0f));
  return y;
}
'''


def test_several_let_chains_lower_to_locals_and_whole_row_chains_are_recognised():
    from tcacomp_b200 import tca
    m = tca.Module(SOFTMAX_BY_STATEMENTS + LAYERNORM_BY_STATEMENTS + TYPED_KERNELS)
    # max | sum of exp | normalise over one x with locals used nowhere else: the one-launch operator replaces them
    assert m.kernels["SoftmaxRows"]["class"] == "softmax_rows"
    d = m.describe("SoftmaxRows")
    assert d["inputs"] == "x" and d["out"] == "y" and d["fused_locals"] == "m,s" and d.get("locals", "") == ""
    assert m.kernels["LayernormRows"]["class"] == "layernorm_rows"
    d = m.describe("LayernormRows")
    assert d["inputs"] == "x,gamma,beta" and d["eps"] == "eps" and d["inv_n"] == "inv_n" and d["fused_locals"] == "mean,var"
    # the typed vocabulary, printed the way the reference's emitter prints it (internal/cg/cxx/naming.go:126-183)
    assert m.describe("ReluSelect") == {"class": "map", "out": "y", "inputs": "x", "map": "((p0 > 0.0f) ? p0 : 0.0f)",
                                        "captures": "", "scalars": ""}
    d = m.describe("CountMultiples")
    assert d["class"] == "chain_reduce" and d["axis"] == "1"
    assert d["map"] == "((((((p0 % 3) == 0) && (p0 != 9)) || ((p0 & 1) == 1)) ? 1.0f : 0.0f) * p1)"
    d = m.describe("BiasRelu")
    assert d["class"] == "map" and d["indexing"] == "0,2" and d["map"] == "static_cast<__nv_bfloat16>(fmaxf((p0 + p1), 0.0f))"
    # the same statements with another epsilon placement are not the recognised group: three launches, the last one a
    # map over five operands
    m3 = tca.Module(LAYERNORM_BY_STATEMENTS.replace("rsqrtf(s2 + eps)", "rsqrtf(eps + s2)"))
    assert m3.kernels["LayernormRows"]["class"] == "chain_reduce+chain_reduce+map"
    assert m3.describe("LayernormRows")["launch2.indexing"] == "0,1,1,2,2"
    # a local that something else reads keeps the statements apart: three launches, two locals to bind
    spread = SOFTMAX_BY_STATEMENTS.replace("expf(v - mx) / sum;", "expf(v - mx) / sum * 2.0f;")
    m2 = tca.Module(spread)
    assert m2.kernels["SoftmaxRows"]["class"] == "chain_reduce+chain_reduce+map"
    d = m2.describe("SoftmaxRows")
    assert d["launches"] == "3" and d["locals"] == "m,s" and d["local.m"] == "f32[R]" and d["launch1.indexing"] == "0,1"
    assert d["launch2.map"] == "((expf((p0 - p1)) / p2) * 2.0f)"
    # a reduction over the middle axis whose map reads the previous reduction's result per output cell
    d = tca.Module(MASKED_NORMALISER_MIDDLE_AXIS).describe("MaskedNormaliser")
    assert d["class"] == "chain_reduce+chain_reduce" and d["locals"] == "m" and d["local.m"] == "f32[7,132]"
    assert d["launch1.axis"] == "1" and d["launch1.indexing"] == "0,3,0" and d["launch1.map"] == "(expf((p0 - p1)) * p2)"
    from tcacomp_b200 import TcabError
    with pytest.raises(TcabError) as e:      # ... but not one that lacks another axis than the reduced one
        tca.Module(MASKED_NORMALISER_MIDDLE_AXIS.replace(
            "on(x[i][k][j], m[i][j], z[i][k][j])", "on(x[i][k][j], m[i][j], z[i][k])").replace(
            "z: tensor<dtype=f32, shape=[7u, 50u, 132u]>", "z: tensor<dtype=f32, shape=[7u, 50u]>")).describe("MaskedNormaliser")
    assert "all but the reduced axis" in e.value.message


def test_include_graph_over_a_file_set():
    from tcacomp_b200 import TcabError, tca
    common = '@name(cxx="Common") kernel common(x: tensor<dtype=f32, shape=[R, C]>) -> tensor<dtype=f32, shape=[R]> {\n' \
             '  dimvar (i, j);\n  let y = map on(x[i][j]) (v: f32): v | reduce(init = 0.0f) on(a: f32, %0: f32) as (i) -> f32: a + %0;\n' \
             '  return y; }\n'
    files = {
        "k/main.tca": '@include "lib/a.tca";\n@include "lib/b.tca";\n' + AFFINE_ROWSUM,
        "k/lib/a.tca": '@include "common.tca";\n' + SCALED_MATMUL,
        "k/lib/b.tca": '@include "common.tca";\n' + BF16_GEMM,          # a diamond: common merges once
        "k/lib/common.tca": common,
    }
    m = tca.Module(files=files, root="k/main.tca")
    # the root's own kernels first, then each include's, depth-first (internal/syntax/module.go:86-124)
    assert m.names() == ["AffineSqRowsum", "ScaledMatmul", "Common", "GemmBiasRelu"]
    cyc = dict(files)
    cyc["k/lib/common.tca"] = '@include "../main.tca";\n' + common
    with pytest.raises(TcabError) as e:
        tca.Module(files=cyc, root="k/main.tca")
    assert "escapes the including file's directory" in e.value.message
    cyc["k/lib/common.tca"] = '@include "a.tca";\n' + common
    with pytest.raises(TcabError) as e:
        tca.Module(files=cyc, root="k/main.tca")
    assert "@include cycle" in e.value.message and "k/lib/common.tca:1:" in e.value.message
    bad = dict(files)
    bad["k/lib/b.tca"] = "kernel oops(\n"
    with pytest.raises(TcabError) as e:
        tca.Module(files=bad, root="k/main.tca")
    assert e.value.message.startswith("k/lib/b.tca:")      # diagnostics of an included file carry its path


def test_launch_argument_checks_need_no_gpu():
    import ctypes as C

    from tcacomp_b200 import _lib, tca
    m = tca.Module(AFFINE_ROWSUM)
    lib = tca.load()
    rc = lib.tcab_module_launch(m._h, b"NoSuchKernel", None, None, 0, None, None, 0, None)
    assert rc == _lib.ERR_INVALID_ARG and b"no kernel named" in lib.tcab_host_last_error()
    # a missing binding is reported by name before anything touches a device
    names = (C.c_char_p * 1)(b"x")
    t = _lib.Tensor()
    t.data, t.dtype, t.rank = 0x1000, _lib.F32, 2
    t.dims[0], t.dims[1] = 8, 8
    tensors = (_lib.Tensor * 1)(t)
    rc = lib.tcab_module_launch(m._h, b"AffineSqRowsum", names, tensors, 1, None, None, 0, None)
    assert rc != _lib.OK
    assert b"y" in lib.tcab_host_last_error() or b"s" in lib.tcab_host_last_error()


@pytest.mark.gpu
def test_text_kernels_on_the_device(oracle, cuda):
    import torch

    from tcacomp_b200 import tca
    m = tca.Module(AFFINE_ROWSUM + SCALED_MATMUL + BF16_GEMM)
    rng = np.random.default_rng(11)

    x = rng.uniform(-1, 1, (1000, 777)).astype(np.float32)
    y = torch.full((1000,), -7.0, device=cuda)
    m.launch("AffineSqRowsum", {"x": torch.from_numpy(x).to(cuda), "y": y}, {"s": 0.5, "t": 0.25})
    from oracle import checks
    assert checks.rowsum_close(y.cpu().numpy(), x)

    lhs = rng.uniform(0, 1, (64, 128)).astype(np.float32)
    rhs = rng.uniform(0, 1, (128, 96)).astype(np.float32)
    out = torch.empty((64, 96), device=cuda)
    m.launch("ScaledMatmul", {"lhs": torch.from_numpy(lhs).to(cuda), "rhs": torch.from_numpy(rhs).to(cuda), "out": out},
             {"scale": 1.5})
    want = oracle.matmul_scale_f32(lhs, rhs, 1.5)
    assert np.abs(out.cpu().numpy() - want).max() <= 1e-5 * np.abs(want).max() * np.sqrt(128)

    a = oracle.f32_to_bf16((rng.normal(0, 1, (300, 264)) / 16).astype(np.float32))
    b = oracle.f32_to_bf16((rng.normal(0, 1, (264, 520)) / 16).astype(np.float32))
    bias = rng.normal(0, 0.02, 520).astype(np.float32)
    dev16 = lambda bits: torch.from_numpy(bits.view(np.int16)).to(cuda).view(torch.bfloat16)  # noqa: E731
    c = torch.empty((300, 520), device=cuda, dtype=torch.bfloat16)
    m.launch("GemmBiasRelu", {"a": dev16(a), "b": dev16(b), "bias": torch.from_numpy(bias).to(cuda), "c": c})
    want = oracle.bf16_to_f32(oracle.gemm_bias_act_bf16(a, b, bias, "relu"))
    got = c.float().cpu().numpy()
    assert np.linalg.norm(got - want) / np.linalg.norm(want) <= 1e-3

    # shape disagreement is reported by dim name, like the generated launcher does
    from tcacomp_b200 import TcabError
    with pytest.raises(TcabError) as e:
        m.launch("ScaledMatmul", {"lhs": torch.empty((64, 128), device=cuda), "rhs": torch.empty((100, 96), device=cuda),
                                  "out": out}, {"scale": 1.0})
    assert e.value.status == 2 and "N" in e.value.message


@pytest.mark.gpu
def test_statement_by_statement_kernels_on_the_device(oracle, cuda):
    import torch

    import tcacomp_b200 as T
    from oracle import checks
    from tcacomp_b200 import tca
    rng = np.random.default_rng(12)
    m = tca.Module(SOFTMAX_BY_STATEMENTS + LAYERNORM_BY_STATEMENTS + TYPED_KERNELS)
    x = (4 * rng.normal(0, 1, (300, 1000))).astype(np.float32)
    xd = torch.from_numpy(x).to(cuda)
    # recognised as a whole: ONE launch, no local bound
    y = torch.empty_like(xd)
    n0 = T.launch_count()
    m.launch("SoftmaxRows", {"x": xd, "y": y})
    assert T.launch_count() - n0 == 1
    assert checks.softmax_close(y.cpu().numpy(), x)
    # kept apart (the last map differs): three launches through locals that the Python host allocates
    m2 = tca.Module(SOFTMAX_BY_STATEMENTS.replace("expf(v - mx) / sum;", "expf(v - mx) / sum * 2.0f;"))
    y2 = torch.empty_like(xd)
    n0 = T.launch_count()
    m2.launch("SoftmaxRows", {"x": xd, "y": y2})
    assert T.launch_count() - n0 == 3
    assert checks.softmax_close(y2.cpu().numpy() * np.float32(0.5), x)
    # locals bound by the caller are used as they are
    mloc, sloc = torch.empty((300,), device=cuda), torch.empty((300,), device=cuda)
    m2.launch("SoftmaxRows", {"x": xd, "y": y2, "m": mloc, "s": sloc})
    assert np.array_equal(mloc.cpu().numpy(), x.max(1))

    # layer-norm by statements on bf16 rows: one launch of the row operator, against the oracle
    xb = oracle.f32_to_bf16(rng.normal(0, 1, (200, 1024)).astype(np.float32))
    g = oracle.f32_to_bf16(rng.normal(1, .1, 1024).astype(np.float32))
    b = oracle.f32_to_bf16(rng.normal(0, .1, 1024).astype(np.float32))
    dev16 = lambda bits: torch.from_numpy(bits.view(np.int16)).to(cuda).view(torch.bfloat16)  # noqa: E731
    yb = torch.empty((200, 1024), device=cuda, dtype=torch.bfloat16)
    n0 = T.launch_count()
    m.launch("LayernormRows", {"x": dev16(xb), "gamma": dev16(g), "beta": dev16(b), "y": yb}, {"inv_n": 1.0 / 1024, "eps": 1e-5})
    assert T.launch_count() - n0 == 1
    assert checks.layernorm_bf16_close(yb.view(torch.int16).cpu().numpy().view(np.uint16), xb, g, b)
    from tcacomp_b200 import TcabError
    with pytest.raises(TcabError) as e:    # the captured factor must be the reciprocal of the row length
        m.launch("LayernormRows", {"x": dev16(xb), "gamma": dev16(g), "beta": dev16(b), "y": yb}, {"inv_n": 0.5, "eps": 1e-5})
    assert "1 / (row length)" in e.value.message

    # middle-axis reduction reading a value per output cell (the local m[i][j]); the Python host allocates m
    mm = tca.Module(MASKED_NORMALISER_MIDDLE_AXIS)
    x3 = (3 * rng.normal(0, 1, (7, 50, 132))).astype(np.float32)
    z3 = rng.uniform(0, 1, (7, 50, 132)).astype(np.float32)
    o3 = torch.empty((7, 132), device=cuda)
    n0 = T.launch_count()
    mm.launch("MaskedNormaliser", {"x": torch.from_numpy(x3).to(cuda), "z": torch.from_numpy(z3).to(cuda), "out": o3})
    assert T.launch_count() - n0 == 2
    want = (np.exp(x3.astype(np.float64) - x3.max(1, keepdims=True)) * z3).sum(1)
    assert (np.abs(o3.cpu().numpy() - want) <= 1e-5 * want).all()

    # typed lambdas from text
    yr = torch.empty_like(xd)
    m.launch("ReluSelect", {"x": xd, "y": yr})
    assert np.array_equal(yr.cpu().numpy(), np.maximum(x, 0))
    k = rng.integers(0, 20, (300, 1000)).astype(np.int32)
    w = rng.uniform(0, 1, (300, 1000)).astype(np.float32)
    n = torch.empty((300,), device=cuda)
    m.launch("CountMultiples", {"k": torch.from_numpy(k).to(cuda), "w": torch.from_numpy(w).to(cuda), "n": n})
    sel = ((k % 3 == 0) & (k != 9)) | ((k & 1) == 1)
    want = (np.where(sel, 1.0, 0.0) * w.astype(np.float64)).sum(1)
    assert (np.abs(n.cpu().numpy() - want) <= 1e-5 * want).all()
    bias = rng.normal(0, 1, 1000).astype(np.float32)
    yb2 = torch.empty((300, 1000), device=cuda, dtype=torch.bfloat16)
    m.launch("BiasRelu", {"x": xd, "bias": torch.from_numpy(bias).to(cuda), "y": yb2})
    want = oracle.f32_to_bf16(np.maximum(x + bias, 0))
    assert np.array_equal(yb2.view(torch.int16).cpu().numpy().view(np.uint16), want)


# ---------------------------------------------------------------------------------------------
# The reference's own suite kernels through this frontend. tests/golden/suite_frontend.json holds what the
# frontend made of testing/kernels/*/*.tca (derived plans, not the sources; tests/golden/make_frontend_golden.py).
# ---------------------------------------------------------------------------------------------
def _frontend_golden():
    import json
    return json.load(open(os.path.join(ROOT, "tests", "golden", "suite_frontend.json")))


# testing/suite.toml tolerances (max abs diff); the kernels it does not list there use the matmul tolerance
FRONTEND_TOL = {"row_sum": 2e-3, "softmax": 2e-3, "transpose": 1e-5, "scale_copy": 1e-5, "axpy3": 1e-5,
                "layernorm": 1e-5, "dup_expr": 1e-5, "dup_const": 1e-5}


def test_frontend_golden_covers_the_suite(oracle):
    golden = _frontend_golden()
    assert sorted(golden) == sorted(oracle.SUITE)
    for name, plan in golden.items():
        cls = oracle.SUITE[name][1]
        assert plan["class"] == ("chain_contract" if cls in ("mm", "qk") else "chain_reduce"), name
        if cls == "qk":
            assert plan["rhs_is_nk"] == "1"
        if cls == "middle":
            assert plan["axis"] == "1"
        if cls == "inner":
            assert plan["axis"] == "2"


def _reference_checkout():
    from oracle.build import REF_DEFAULT
    return os.environ.get("TCAB_REFERENCE", REF_DEFAULT)


def test_frontend_golden_is_reproducible():
    if not os.path.isdir(os.path.join(_reference_checkout(), "testing", "kernels")):
        pytest.skip("needs the reference checkout")
    import importlib.util
    spec = importlib.util.spec_from_file_location("make_frontend_golden",
                                                  os.path.join(ROOT, "tests", "golden", "make_frontend_golden.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    assert mod.derive(_reference_checkout()) == _frontend_golden()


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["axpy3", "dup_const", "dup_expr", "gemm", "layernorm", "mlp", "mm_mid", "mm_small",
                                  "mm_splitk", "qk_score", "row_sum", "scale_copy", "softmax", "transpose"])
def test_reference_kernel_text_to_numbers(oracle, cuda, name):
    # reference kernel text -> (this frontend, at fixture time) -> plan -> device -> the oracle's restatement of the
    # reference's runner for that kernel
    import torch

    import tcacomp_b200 as T
    plan = _frontend_golden()[name]
    x, z = oracle.suite_inputs(name)
    want = oracle.suite(name)
    declared = [s for s in plan["scalars"].split(",") if s]
    values = dict(zip(declared, oracle.SUITE[name][3]))
    caps = tuple(values[c] for c in plan["captures"].split(",") if c)
    xd, zd = torch.from_numpy(x).to(cuda), torch.from_numpy(z).to(cuda)
    post = plan["post"] or None
    if plan["class"] == "chain_reduce":
        got = T.chain_reduce([xd, zd], plan["map"], combine_expr=plan["combine"], init=float(plan["init"]),
                             post_expr=post, captures=caps, axis=int(plan["axis"]))
    else:
        got = T.chain_contract(xd, zd, plan["map"], rhs_is_nk=plan["rhs_is_nk"] == "1", combine_expr=plan["combine"],
                               init=float(plan["init"]), post_expr=post, captures=caps)
    got = got.cpu().numpy()
    assert got.shape == want.shape
    assert np.abs(got.astype(np.float64) - want).max() <= FRONTEND_TOL.get(name, 2e-3)
