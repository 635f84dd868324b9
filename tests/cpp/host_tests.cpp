// host_tests.cpp -- tests of the C++ builder mirror, written the way the reference tests its own
// builder and kernels:
//   * the CPU half follows pkg/builder_test.go (eager checks, typestate, deferred errors) and
//     pkg/oracle_test.go (the matmul_scale chain builds), with a CHECK macro like
//     runtime/tests/cpu_tests.cpp;
//   * the GPU half (--gpu) follows testing/runners/*.cu: deterministic inputs elem(i), a canary in
//     the output, an in-binary naive fp32 CPU loop, and the protocol lines
//     KERNEL / CANARY / CHECKSUM / REF_CHECKSUM / MAXDIFF that the caller parses.
#include <cmath>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#include "../../tcacomp_b200/csrc/host/pkg.h"
#include "../../tcacomp_b200/csrc/host/pkg_ext.h"
#include "../../tcacomp_b200/csrc/host/tca_syntax.h"
#include "../../include/tcab_tuning.h"

#ifdef HOST_TESTS_WITH_CUDA
#include <cuda_runtime.h>
#endif

using namespace tcab::pkg;

static int g_checks = 0, g_failures = 0;
#define CHECK(cond)                                                    \
  do {                                                                 \
    ++g_checks;                                                        \
    if (!(cond)) {                                                     \
      ++g_failures;                                                    \
      std::printf("FAIL %s:%d: %s\n", __FILE__, __LINE__, #cond);      \
    }                                                                  \
  } while (0)

static bool contains(const std::string& s, const char* what) { return s.find(what) != std::string::npos; }

// ---------------------------------------------------------------------------------------------
// CPU half
// ---------------------------------------------------------------------------------------------
static void oracle_dims(Builder& b, Dim* m, Dim* k, Dim* n) {
  *m = b.Dim("m", 0);
  *k = b.Dim("k", 0);
  *n = b.Dim("n", 0);
}

// pkg/oracle_test.go:17-63: out[m,k] = scale * sum_n lhs[m,n] * rhs[n,k]
static void test_matmul_scale_builds() {
  Builder b("matmul_scale");
  Dim m, k, n;
  oracle_dims(b, &m, &k, &n);
  Tensor lhs = b.Tensor("lhs", Elem::F32, m, n), rhs = b.Tensor("rhs", Elem::F32, n, k);
  Tensor out = b.Tensor("output", Elem::F32, m, k);
  Expr scale = b.ScalarParam("scale", Elem::F32);
  auto root = b.Stmt().Iter(m, k, n).Map({At(lhs, m, n), At(rhs, n, k)}, [&](Expr l, Expr r) { return b.Mul(l, r); });
  CHECK(root.ok());
  auto mid = root.value.As(m, k, n);
  auto ar = mid.Reduce(b.Float32(0.0f), [&](Expr acc, Expr v) { return b.Add(acc, v); });
  CHECK(ar.ok());
  auto am = ar.value.Map({}, [&](Expr v) { return b.Mul(v, scale); });
  CHECK(am.ok());
  auto st = am.value.As(m, k).Store(out, m, k);
  CHECK(st.ok());
  auto g = b.Build();
  CHECK(g.ok());
  CHECK(g.value.statements.size() == 1);
  // a contraction of fp32 operands: lhs[m,n] with rhs[n,k], reduced over n, piped scale
  auto plan = Classify(g.value.statements[0]);
  CHECK(plan.ok() && plan.value.kind == Plan::ChainContract && !plan.value.rhs_is_nk);
  CHECK(plan.value.map_expr == "(p0 * p1)" && plan.value.post_expr == "(p0 * c0)");
  CHECK(plan.value.capture_names.size() == 1 && plan.value.capture_names[0] == "scale");
}

// pkg/builder_test.go:21-160
static void test_eager_checks() {
  {  // wrongMapArity
    Builder b("arity");
    Dim m, k, n;
    oracle_dims(b, &m, &k, &n);
    Tensor lhs = b.Tensor("lhs", Elem::F32, m, n), rhs = b.Tensor("rhs", Elem::F32, n, k);
    auto r = b.Stmt().Iter(m, k, n).Map({At(lhs, m, n), At(rhs, n, k)}, [&](Expr l) { return l; });
    CHECK(!r.ok() && contains(r.err, "arity"));
  }
  {  // wrongPipedMapArity
    Builder b("arity-piped");
    Dim m, k, n;
    oracle_dims(b, &m, &k, &n);
    Tensor lhs = b.Tensor("lhs", Elem::F32, m, n);
    auto ra = b.Stmt().Iter(m, k, n).Map({At(lhs, m, n)}, [&](Expr v) { return v; });
    CHECK(ra.ok());
    auto ar = ra.value.As(m, k, n).Reduce(b.Float32(0), [&](Expr a, Expr v) { return b.Add(a, v); });
    CHECK(ar.ok());
    auto am = ar.value.Map({}, [&](Expr a, Expr) { return a; });
    CHECK(!am.ok() && contains(am.err, "arity"));
  }
  {  // duplicateAxisInAs: surfaces at the next rung and names the missing axis
    Builder b("dup-as");
    Dim m, k, n;
    oracle_dims(b, &m, &k, &n);
    Tensor lhs = b.Tensor("lhs", Elem::F32, m, n), rhs = b.Tensor("rhs", Elem::F32, n, k);
    auto ra = b.Stmt().Iter(m, k, n).Map({At(lhs, m, n), At(rhs, n, k)}, [&](Expr l, Expr r) { return b.Mul(l, r); });
    CHECK(ra.ok());
    auto red = ra.value.As(m, k, k).Reduce(b.Float32(0), [&](Expr a, Expr v) { return b.Add(a, v); });
    CHECK(!red.ok() && contains(red.err, "@n"));
  }
  {  // omitLiveAxisInAs
    Builder b("omit-as");
    Dim m, k, n;
    oracle_dims(b, &m, &k, &n);
    Tensor lhs = b.Tensor("lhs", Elem::F32, m, n);
    auto ra = b.Stmt().Iter(m, k, n).Map({At(lhs, m, n)}, [&](Expr l) { return l; });
    CHECK(ra.ok());
    auto red = ra.value.As(m).Reduce(b.Float32(0), [&](Expr a, Expr v) { return b.Add(a, v); });
    CHECK(!red.ok());
  }
  {  // heterogeneousReducer
    Builder b("hetero-reduce");
    Dim m, k, n;
    oracle_dims(b, &m, &k, &n);
    Tensor lhs = b.Tensor("lhs", Elem::F32, m, n);
    auto ra = b.Stmt().Iter(m, k, n).Map({At(lhs, m, n)}, [&](Expr l) { return l; });
    CHECK(ra.ok());
    auto red = ra.value.As(m, k, n).Reduce(b.Int32(0), [&](Expr a, Expr v) { return b.Add(a, v); });
    CHECK(!red.ok() && contains(red.err, "homogeneous"));
  }
  {  // wrongSubscriptCount
    Builder b("subscripts");
    Dim m, k, n;
    oracle_dims(b, &m, &k, &n);
    Tensor lhs = b.Tensor("lhs", Elem::F32, m, n), rhs = b.Tensor("rhs", Elem::F32, n, k);
    auto r = b.Stmt().Iter(m, k, n).Map({At(lhs, m), At(rhs, n, k)}, [&](Expr l, Expr r2) { return b.Mul(l, r2); });
    CHECK(!r.ok() && contains(r.err, "rank"));
  }
  {  // undeclaredDim: a dim from another builder
    Builder b("undeclared"), other("other");
    Dim m, k, n;
    oracle_dims(b, &m, &k, &n);
    Tensor lhs = b.Tensor("lhs", Elem::F32, m, n), rhs = b.Tensor("rhs", Elem::F32, n, k);
    Dim foreign = other.Dim("z", 0);
    auto r = b.Stmt().Iter(m, k, n).Map({At(lhs, m, foreign), At(rhs, n, k)},
                                         [&](Expr l, Expr r2) { return b.Mul(l, r2); });
    CHECK(!r.ok() && contains(r.err, "declared"));
  }
  {  // unknownBuiltin
    Builder b("builtin");
    Expr e = b.Call("threadIdx_x", {});
    CHECK(!e.ok() && contains(e.err, "unknown builtin"));
  }
  {  // badOperandAxis
    Builder b("operand-axis");
    Dim m, k, n;
    oracle_dims(b, &m, &k, &n);
    Tensor lhs = b.Tensor("lhs", Elem::F32, m, n);
    auto r = b.Stmt().Iter(m, k, n).Map({At(lhs, m, k)}, [&](Expr l) { return l; });
    CHECK(!r.ok() && contains(r.err, "dim"));
  }
  {  // no implicit promotion (pkg/expr.go:137-176); the error travels inside the Expr to the rung
    Builder b("promo");
    Dim m = b.Dim("m", 0), n = b.Dim("n", 0);
    Tensor x = b.Tensor("x", Elem::F32, m, n);
    auto r = b.Stmt().Iter(m, n).Map({At(x, m, n)}, [&](Expr v) { return b.Add(v, b.Int32(1)); });
    CHECK(!r.ok() && contains(r.err, "implicit promotions"));
  }
  {  // declaration errors are deferred to the next error-returning rung, or to Build (pkg/builder.go:22-27)
    Builder b("deferred");
    Dim m = b.Dim("m", 0);
    b.Dim("m", 4);  // duplicate: no error here
    Dim n = b.Dim("n", -3);
    (void)n;
    auto g = b.Build();
    CHECK(!g.ok() && contains(g.err, "already declared"));
    Builder b2("deferred2");
    Dim m2 = b2.Dim("m", 0), n2 = b2.Dim("n", 0);
    b2.Dim("n", 0);
    Tensor x = b2.Tensor("x", Elem::F32, m2, n2);
    auto r = b2.Stmt().Iter(m2, n2).Map({At(x, m2, n2)}, [&](Expr v) { return v; });
    CHECK(!r.ok() && contains(r.err, "already declared"));
    (void)m;
  }
  {  // a chain that was never stored fails Build
    Builder b("unstored");
    Dim m = b.Dim("m", 0), n = b.Dim("n", 0);
    Tensor x = b.Tensor("x", Elem::F32, m, n);
    auto r = b.Stmt().Iter(m, n).Map({At(x, m, n)}, [&](Expr v) { return v; });
    CHECK(r.ok());
    auto g = b.Build();
    CHECK(!g.ok() && contains(g.err, "never stored"));
  }
}

// pkg/builder_test.go:162-: every legal rung sequence (the illegal ones do not compile)
static void test_typestate_and_classification() {
  {  // reduceThenStore: y[i] = sum_j (0.5*x+0.25)^2  -> the chain class, innermost axis
    Builder b("c1");
    Dim i = b.Dim("i", 0), j = b.Dim("j", 0);
    Tensor x = b.Tensor("x", Elem::F32, i, j), y = b.Tensor("y", Elem::F32, i);
    auto ra = b.Stmt().Iter(i, j).Map({At(x, i, j)}, [&](Expr v) {
      Expr t = b.Add(b.Mul(b.Float32(0.5f), v), b.Float32(0.25f));
      return b.Mul(t, t);
    });
    CHECK(ra.ok());
    auto ar = ra.value.As(i, j).Reduce(b.Float32(0), [&](Expr a, Expr v) { return b.Add(a, v); });
    CHECK(ar.ok());
    CHECK(ar.value.Store(y, i).ok());
    auto g = b.Build();
    CHECK(g.ok());
    auto p = Classify(g.value.statements[0]);
    CHECK(p.ok() && p.value.kind == Plan::ChainReduce && p.value.reduce_axis == 1);
    CHECK(p.value.map_expr == "(((0.5f * p0) + 0.25f) * ((0.5f * p0) + 0.25f))");
    CHECK(p.value.combine_expr == "(p0 + p1)" && p.value.post_expr.empty());
  }
  {  // middle-axis reduce with a piped map and scalar captures (the suite's axpy3 shape)
    Builder b("axpy3");
    Dim i = b.Dim("i", 0), k = b.Dim("k", 4), j = b.Dim("j", 0);
    Tensor x = b.Tensor("x", Elem::F32, i, k, j), z = b.Tensor("z", Elem::F32, i, k, j);
    Tensor out = b.Tensor("out", Elem::F32, i, j);
    Expr alpha = b.ScalarParam("alpha", Elem::F32), beta = b.ScalarParam("beta", Elem::F32);
    Expr gamma = b.ScalarParam("gamma", Elem::F32);
    auto ra = b.Stmt().Iter(i, k, j).Map({At(x, i, k, j), At(z, i, k, j)}, [&](Expr xv, Expr zv) {
      return b.Add(b.Mul(alpha, xv), b.Mul(beta, zv));
    });
    CHECK(ra.ok());
    auto ar = ra.value.As(i, j, k).Reduce(b.Float32(0), [&](Expr a, Expr v) { return b.Add(a, v); });
    CHECK(ar.ok());
    auto am = ar.value.Map({}, [&](Expr v) { return b.Add(v, b.Mul(gamma, b.Call("tanhf", {v}))); });
    CHECK(am.ok());
    CHECK(am.value.As(i, j).Store(out, i, j).ok());
    auto g = b.Build();
    CHECK(g.ok());
    auto p = Classify(g.value.statements[0]);
    CHECK(p.ok() && p.value.reduce_axis == 1);
    CHECK(p.value.map_expr == "((c0 * p0) + (c1 * p1))" && p.value.post_expr == "(p0 + (c2 * tanhf(p0)))");
    CHECK(p.value.capture_names.size() == 3 && p.value.capture_names[2] == "gamma");
  }
  {  // chainedReductions build; the kernel library reduces one axis per launch
    Builder b("two-reduce");
    Dim m = b.Dim("m", 0), k = b.Dim("k", 0), n = b.Dim("n", 0);
    Tensor x = b.Tensor("x", Elem::F32, m, k, n), o = b.Tensor("o", Elem::F32, m);
    auto ra = b.Stmt().Iter(m, k, n).Map({At(x, m, k, n)}, [&](Expr v) { return v; });
    auto ar = ra.value.As(m, k, n).Reduce(b.Float32(0), [&](Expr a, Expr v) { return b.Add(a, v); });
    auto ar2 = ar.value.Reduce(b.Float32(0), [&](Expr a, Expr v) { return b.Add(a, v); });
    CHECK(ar2.ok() && ar2.value.Store(o, m).ok());
    auto g = b.Build();
    CHECK(g.ok());
    CHECK(!Classify(g.value.statements[0]).ok());
  }
  {  // the bf16 contraction with bias and ReLU -> the contraction class
    Builder b("gemm");
    Dim m = b.Dim("m", 0), n = b.Dim("n", 0), k = b.Dim("k", 0);
    Tensor A = b.Tensor("a", Elem::BF16, m, k), B = b.Tensor("b", Elem::BF16, k, n);
    Tensor bias = b.Tensor("bias", Elem::F32, n), C = b.Tensor("c", Elem::BF16, m, n);
    auto ra = b.Stmt().Iter(m, n, k).Map({At(A, m, k), At(B, k, n)}, [&](Expr l, Expr r) {
      return b.Mul(b.Cast(l, Elem::F32), b.Cast(r, Elem::F32));
    });
    CHECK(ra.ok());
    auto ar = ra.value.As(m, n, k).Reduce(b.Float32(0), [&](Expr a, Expr v) { return b.Add(a, v); });
    CHECK(ar.ok());
    auto am = ar.value.Map({At(bias, n)}, [&](Expr v, Expr bb) {
      return b.Cast(b.Call("fmaxf", {b.Add(v, bb), b.Float32(0)}), Elem::BF16);
    });
    CHECK(am.ok());
    CHECK(am.value.As(m, n).Store(C, m, n).ok());
    auto g = b.Build();
    CHECK(g.ok());
    auto p = Classify(g.value.statements[0]);
    CHECK(p.ok() && p.value.kind == Plan::GemmBiasAct && p.value.act == TCAB_ACT_RELU && p.value.bias == "bias");
  }
  {  // the generated launcher's shape contract, by name, before anything is launched
    Builder b("shapes");
    Dim i = b.Dim("i", 0), j = b.Dim("j", 0);
    Tensor x = b.Tensor("x", Elem::F32, i, j), y = b.Tensor("y", Elem::F32, i);
    auto ra = b.Stmt().Iter(i, j).Map({At(x, i, j)}, [&](Expr v) { return v; });
    auto ar = ra.value.As(i, j).Reduce(b.Float32(0), [&](Expr a, Expr v) { return b.Add(a, v); });
    CHECK(ar.value.Store(y, i).ok());
    auto g = b.Build();
    Bindings bind;
    tcab_tensor tx{reinterpret_cast<void*>(0x1000), TCAB_F32, 2, {8, 16, 0, 0}};
    tcab_tensor ty{reinterpret_cast<void*>(0x2000), TCAB_F32, 1, {9, 0, 0, 0}};
    bind.tensors["x"] = tx;
    bind.tensors["y"] = ty;
    CHECK(Launch(g.value, bind, nullptr) == TCAB_ERR_SHAPE && contains(LastError(), "y.Dim(0) must equal i"));
    bind.tensors.erase("y");
    CHECK(Launch(g.value, bind, nullptr) == TCAB_ERR_INVALID_ARG && contains(LastError(), "not bound"));
  }
}

// ---------------------------------------------------------------------------------------------
// The .tca text frontend (internal/syntax/parser/parser_test.go, internal/syntax/semacheck tests and
// internal/e2e/frontend_test.go cover the same ground in the reference): texts written for this test.
// ---------------------------------------------------------------------------------------------
static const char* kTcaWeightedFold = R"tca(
// out[i][j] = bump + lift * sum_k (w0 * x + w1 * z), the trailing extent a compile-time constant
@runtime(cxx_path="runtime/tca_runtime.h");
@name(cxx="WeightedFold")
kernel weighted_fold(
  x: tensor<dtype=f32, shape=[R, C, 8u]>,
  z: tensor<dtype=f32, shape=[R, C, 8u]>,
  w0: f32, w1: f32, lift: f32,
) -> tensor<dtype=f32, shape=[R, C]>
{
  dimvar (i, j, k);
  let folded = map
    on(x[i][j][k], z[i][j][k])
    [w0, w1] (a: f32, b: f32) -> f32:
      w0 * a + w1 * b
  | reduce(init = 0.0f)
    on(acc: f32, %0: f32)
    as (i, j) -> f32:
      acc + %0
  | map
    on()
    [lift] (s: f32) -> f32:
      0.25f + lift * s   /* literal lifted into a capture slot */
  ;
  return folded;
}
)tca";

static const char* kTcaMidAxis = R"tca(
@name(cxx="MidAxisMax")
kernel mid_axis_max(x: tensor<dtype=f32, shape=[B, 6u, C]>) -> tensor<dtype=f32, shape=[B, C]> {
  dimvar b, k, c;
  let m = map on(x[b][k][c]) (v: f32): v * v - 0.5f
        | reduce(init = -inf_f32) on(best: f32, %0) as (b, c) -> f32: fmaxf(best, %0);
  return m;
}
)tca";

static const char* kTcaScores = R"tca(
@name(cxx="Scores")
kernel scores(q: tensor<dtype=f32, shape=[H, D]>, keys: tensor<dtype=f32, shape=[N, D]>, temp: f32)
    -> tensor<dtype=f32, shape=[H, N]> {
  dimvar (h, n, d);
  let s = map on(q[h][d], keys[n][d]) (l: f32, r: f32) -> f32: l * r
        | reduce(init = 0.0f) on(acc: f32, %0: f32) as (h, n) -> f32: acc + %0
        | map on() [temp] (v: f32) -> f32: v * temp;
  return s;
}
)tca";

static std::string tca_error(const std::string& text) {
  auto r = ParseModule(text);
  return r.ok() ? std::string("<accepted>") : r.err;
}

static void test_tca_frontend() {
  {
    auto r = ParseModule(kTcaWeightedFold);
    CHECK(r.ok());
    if (!r.ok()) std::printf("  %s\n", r.err.c_str());
    CHECK(r.value.size() == 1);
    if (r.ok() && r.value.size() == 1) {
      const ParsedKernel& pk = r.value[0];
      CHECK(pk.name == "weighted_fold" && pk.cxx_name == "WeightedFold" && pk.output == "folded");
      CHECK(pk.graph.statements.size() == 1);
      auto plan = Classify(pk.graph.statements[0]);
      CHECK(plan.ok() && plan.value.kind == Plan::ChainReduce && plan.value.reduce_axis == 2);
      CHECK(plan.value.map_expr == "((c0 * p0) + (c1 * p1))");
      CHECK(plan.value.combine_expr == "(p0 + p1)");
      CHECK(contains(plan.value.post_expr, "* p0") && contains(plan.value.post_expr, "0.25"));
      CHECK(plan.value.capture_names.size() >= 3 && plan.value.capture_names[0] == "w0" && plan.value.capture_names[1] == "w1");
    }
  }
  {
    auto r = ParseModule(kTcaMidAxis);
    CHECK(r.ok());
    if (!r.ok()) std::printf("  %s\n", r.err.c_str());
    if (r.ok()) {
      auto plan = Classify(r.value[0].graph.statements[0]);
      CHECK(plan.ok() && plan.value.kind == Plan::ChainReduce && plan.value.reduce_axis == 1);
      CHECK(plan.value.combine_expr == "fmaxf(p0, p1)" && std::isinf(plan.value.init) && plan.value.init < 0);
    }
  }
  {
    auto r = ParseModule(std::string(kTcaScores) + kTcaMidAxis);  // two kernels in one module
    CHECK(r.ok() && r.value.size() == 2);
    if (!r.ok()) std::printf("  %s\n", r.err.c_str());
    if (r.ok()) {
      auto plan = Classify(r.value[0].graph.statements[0]);
      CHECK(plan.ok() && plan.value.kind == Plan::ChainContract && plan.value.rhs_is_nk);
      CHECK(plan.value.post_expr == "(p0 * c0)" && plan.value.capture_names.size() == 1 && plan.value.capture_names[0] == "temp");
      CHECK(r.value[1].cxx_name == "MidAxisMax");
    }
  }
  // diagnostics carry line:col (internal/syntax/parser/parser.go error positions)
  CHECK(contains(tca_error("kernel k(x: tensor<dtype=f32, shape=[R, 4]>) -> f32 { }"), "1:41: a constant extent is an unsigned literal"));
  CHECK(contains(tca_error("kernel k(x: tensor<dtype=f64, shape=[R]>) -> f32 { }"), "1:"));
  // a conditional is typed like pkg/expr.go:271 Select: bool condition, branches of one type
  CHECK(contains(tca_error("kernel k(x: tensor<dtype=f32, shape=[R, C]>) -> tensor<dtype=f32, shape=[R]> {\n"
                           "  dimvar (i, j);\n"
                           "  let o = map on(x[i][j]) (v: f32): v > 0.0f ? v : 0.0f\n"
                           "    | reduce(init = 0.0f) on(a: f32, %0) as (i) -> f32: a + %0;\n  return o; }"),
                 "<accepted>"));
  CHECK(contains(tca_error("kernel k(x: tensor<dtype=f32, shape=[R, C]>) -> tensor<dtype=f32, shape=[R]> {\n"
                           "  dimvar (i, j);\n"
                           "  let o = map on(x[i][j]) (v: f32): v ? v : 0.0f\n"
                           "    | reduce(init = 0.0f) on(a: f32, %0) as (i) -> f32: a + %0;\n  return o; }"),
                 "3:11: select: condition must be bool"));
  // a map alone is stored through the added rung (pkg_ext.h; the reference requires a reduction, pkg/chain.go:433-438);
  // a second map still needs a reduction before it
  CHECK(contains(tca_error("kernel k(x: tensor<dtype=f32, shape=[R, C]>) -> tensor<dtype=f32, shape=[R, C]> {\n"
                           "  dimvar (i, j);\n  let o = map on(x[i][j]) (v: f32): v + 1.0f;\n  return o; }"),
                 "<accepted>"));
  CHECK(contains(tca_error("kernel k(x: tensor<dtype=f32, shape=[R, C]>) -> tensor<dtype=f32, shape=[R, C]> {\n"
                           "  dimvar (i, j);\n  let o = map on(x[i][j]) (v: f32): v + 1.0f | map on() (w: f32): w;\n  return o; }"),
                 "a second map needs a reduction before it"));
  // arity, unknown names, uncaptured scalars, rank and dimvar consistency (semacheck rules of section 7)
  const std::string head = "kernel k(x: tensor<dtype=f32, shape=[R, C]>, y: tensor<dtype=f32, shape=[C, R]>, g: f32) -> tensor<dtype=f32, shape=[R]> {\n  dimvar (i, j);\n";
  const std::string fold = "\n    | reduce(init = 0.0f) on(a: f32, %0) as (i) -> f32: a + %0;\n  return o; }";
  CHECK(contains(tca_error(head + "  let o = map on(x[i][j]) (v: f32, w: f32): v * w" + fold), "3:11: root map: 2 lambda parameters for 1 operands"));
  CHECK(contains(tca_error(head + "  let o = map on(x[i][j]) (v: f32): v * q" + fold), "unknown name 'q'"));
  CHECK(contains(tca_error(head + "  let o = map on(x[i][j]) (v: f32): v * g" + fold), "used but not captured"));
  CHECK(contains(tca_error(head + "  let o = map on(x[i][j]) [g] (v: f32): v * g" + fold), "<accepted>"));
  CHECK(contains(tca_error(head + "  let o = map on(x[i]) (v: f32): v" + fold), "has rank 2, subscripted with 1"));
  CHECK(contains(tca_error(head + "  let o = map on(x[i][j], y[i][j]) (v: f32, w: f32): v * w" + fold), "one extent per dimvar"));
  CHECK(contains(tca_error(head + "  let o = map on(x[i][t]) (v: f32): v" + fold), "'t' is not a declared dimvar"));
  CHECK(contains(tca_error(head + "  let o = map on(x[i][j]) (v: f32): v" + fold.substr(0, fold.find("return")) + "return x; }"), "'return' must name a let-bound tensor"));
  CHECK(contains(tca_error(head + "  let o = map on(x[i][j]) (v: f32): powf(v)" + fold), "powf"));
  CHECK(contains(tca_error("@include \"other.tca\";"), "1:10: missing include file \"other.tca\""));
  CHECK(contains(tca_error("kernel k(x: tensor<dtype=f32, shape=[R]>) -> f32 { let o = map on(x[i]) (v: f32): v /* open"), "unterminated"));
}

// ---------------------------------------------------------------------------------------------
// GPU half: the reference's runner protocol (testing/runners/common.cuh)
// ---------------------------------------------------------------------------------------------
#ifdef HOST_TESTS_WITH_CUDA

static float elem(unsigned i) { return static_cast<float>((i * 2654435761u) % 1000u) / 1000.0f; }

static uint16_t f2bf(float f) {
  uint32_t u;
  std::memcpy(&u, &f, 4);
  u += 0x7fffu + ((u >> 16) & 1u);
  return static_cast<uint16_t>(u >> 16);
}
static float bf2f(uint16_t h) {
  uint32_t u = static_cast<uint32_t>(h) << 16;
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}

#define CUDA_OK(call)                                      \
  do {                                                     \
    if ((call) != cudaSuccess) {                           \
      std::printf("CUDA_FAIL %s:%d\n", __FILE__, __LINE__); \
      return false;                                        \
    }                                                      \
  } while (0)

struct DeviceBuf {
  void* p = nullptr;
  ~DeviceBuf() { cudaFree(p); }
};

// Uploads, launches the graph, downloads `out_name`, prints the protocol lines against `ref`.
static bool run_and_report(const char* kernel, const Graph& g, std::vector<std::pair<std::string, tcab_tensor>> tensors,
                           const std::vector<const void*>& host_data, const std::map<std::string, float>& scalars,
                           const std::string& out_name, const std::vector<float>& ref, bool out_bf16) {
  Bindings bind;
  bind.scalars = scalars;
  std::vector<DeviceBuf> bufs(tensors.size());
  size_t out_index = 0, out_elems = 0;
  for (size_t i = 0; i < tensors.size(); ++i) {
    tcab_tensor& t = tensors[i].second;
    size_t n = 1;
    for (uint32_t d = 0; d < t.rank; ++d) n *= t.dims[d];
    const size_t bytes = n * (t.dtype == TCAB_BF16 ? 2 : 4);
    CUDA_OK(cudaMalloc(&bufs[i].p, bytes ? bytes : 4));
    if (tensors[i].first == out_name) {
      out_index = i;
      out_elems = n;
      if (out_bf16) {
        std::vector<uint16_t> canary(n, f2bf(-12345.0f));
        CUDA_OK(cudaMemcpy(bufs[i].p, canary.data(), bytes, cudaMemcpyHostToDevice));
      } else {
        std::vector<float> canary(n, -12345.0f);
        CUDA_OK(cudaMemcpy(bufs[i].p, canary.data(), bytes, cudaMemcpyHostToDevice));
      }
    } else {
      CUDA_OK(cudaMemcpy(bufs[i].p, host_data[i], bytes, cudaMemcpyHostToDevice));
    }
    t.data = bufs[i].p;
    bind.tensors[tensors[i].first] = t;
  }
  const int rc = Launch(g, bind, nullptr);
  if (rc != TCAB_OK) {
    std::printf("KERNEL %s\nLAUNCH_FAIL %d %s\n", kernel, rc, LastError().c_str());
    return false;
  }
  CUDA_OK(cudaDeviceSynchronize());
  std::vector<float> got(out_elems);
  if (out_bf16) {
    std::vector<uint16_t> raw(out_elems);
    CUDA_OK(cudaMemcpy(raw.data(), bufs[out_index].p, out_elems * 2, cudaMemcpyDeviceToHost));
    for (size_t i = 0; i < out_elems; ++i) got[i] = bf2f(raw[i]);
  } else {
    CUDA_OK(cudaMemcpy(got.data(), bufs[out_index].p, out_elems * 4, cudaMemcpyDeviceToHost));
  }
  unsigned canary = 0;
  double gsum = 0, rsum = 0, maxdiff = 0;
  const float cval = out_bf16 ? bf2f(f2bf(-12345.0f)) : -12345.0f;
  for (size_t i = 0; i < out_elems; ++i) {
    if (got[i] == cval) ++canary;
    gsum += got[i];
    rsum += ref[i];
    const double d = std::fabs(static_cast<double>(got[i]) - static_cast<double>(ref[i]));
    if (d > maxdiff) maxdiff = d;
  }
  std::printf("KERNEL %s\nCANARY %u\nCHECKSUM %.17g\nREF_CHECKSUM %.17g\nMAXDIFF %.17g\n", kernel, canary, gsum, rsum,
              maxdiff);
  return true;
}

static tcab_tensor view(int dtype, std::vector<uint32_t> dims) {
  tcab_tensor t;
  std::memset(&t, 0, sizeof(t));
  t.dtype = dtype;
  t.rank = static_cast<uint32_t>(dims.size());
  for (size_t i = 0; i < dims.size(); ++i) t.dims[i] = dims[i];
  return t;
}

// A suite kernel whose operands x, z are [d0, d1, d2] reduced over `axis` (1 or 2) with a map of two
// operands, built through the rungs like the .tca source declares it.
static bool suite_case(const char* name, unsigned d0, unsigned d1, unsigned d2, int axis,
                       const std::function<Expr(Builder&, Expr, Expr, std::map<std::string, Expr>&)>& map_fn,
                       const std::function<Expr(Builder&, Expr)>& post_fn, const std::map<std::string, float>& scalars,
                       const std::function<float(float, float)>& cpu_map, const std::function<float(float)>& cpu_post) {
  Builder b(name);
  Dim a0 = b.Dim("i", 0), a1 = b.Dim(axis == 1 ? "k" : "j", 0), a2 = b.Dim(axis == 1 ? "j" : "k", 0);
  Tensor x = b.Tensor("x", Elem::F32, a0, a1, a2), z = b.Tensor("z", Elem::F32, a0, a1, a2);
  Dim keep = axis == 1 ? a2 : a1, red = axis == 1 ? a1 : a2;
  Tensor out = b.Tensor("out", Elem::F32, a0, keep);
  std::map<std::string, Expr> sp;  // scalar parameters, declared once (pkg/builder.go:285-295)
  for (const auto& s : scalars) sp[s.first] = b.ScalarParam(s.first, Elem::F32);
  auto ra = b.Stmt().Iter(a0, a1, a2).Map({At(x, a0, a1, a2), At(z, a0, a1, a2)},
                                           [&](Expr v, Expr w) { return map_fn(b, v, w, sp); });
  if (!ra.ok()) { std::printf("BUILD_FAIL %s: %s\n", name, ra.err.c_str()); return false; }
  auto ar = ra.value.As(a0, keep, red).Reduce(b.Float32(0.0f), [&](Expr acc, Expr v) { return b.Add(acc, v); });
  if (!ar.ok()) { std::printf("BUILD_FAIL %s: %s\n", name, ar.err.c_str()); return false; }
  Result<Stored> st;
  if (post_fn) {
    auto am = ar.value.Map({}, [&](Expr v) { return post_fn(b, v); });
    if (!am.ok()) { std::printf("BUILD_FAIL %s: %s\n", name, am.err.c_str()); return false; }
    st = am.value.As(a0, keep).Store(out, a0, keep);
  } else {
    st = ar.value.Store(out, a0, keep);
  }
  auto g = b.Build();
  if (!st.ok() || !g.ok()) { std::printf("BUILD_FAIL %s: %s%s\n", name, st.err.c_str(), g.err.c_str()); return false; }

  const unsigned n = d0 * d1 * d2;
  std::vector<float> hx(n), hz(n);
  for (unsigned i = 0; i < n; ++i) hx[i] = hz[i] = elem(i);
  const unsigned dk = axis == 1 ? d1 : d2, dc = axis == 1 ? d2 : d1;
  std::vector<float> ref(static_cast<size_t>(d0) * dc);
  for (unsigned i = 0; i < d0; ++i)
    for (unsigned j = 0; j < dc; ++j) {
      float acc = 0.0f;
      for (unsigned k = 0; k < dk; ++k) {
        const size_t o = axis == 1 ? (static_cast<size_t>(i) * dk + k) * dc + j : (static_cast<size_t>(i) * dc + j) * dk + k;
        acc += cpu_map(hx[o], hz[o]);
      }
      ref[static_cast<size_t>(i) * dc + j] = cpu_post ? cpu_post(acc) : acc;
    }
  return run_and_report(name, g.value,
                        {{"x", view(TCAB_F32, {d0, d1, d2})}, {"z", view(TCAB_F32, {d0, d1, d2})},
                         {"out", view(TCAB_F32, {d0, dc})}},
                        {hx.data(), hz.data(), nullptr}, scalars, "out", ref, false);
}

static bool gpu_tests() {
  bool ok = true;
  // testing/kernels/runtime/row_sum.tca, testing/runners/row_sum.cu
  ok &= suite_case("RowSum", 512, 4, 1024, 1, [](Builder& b, Expr v, Expr w, std::map<std::string, Expr>&) { return b.Mul(v, w); }, nullptr, {},
                   [](float v, float w) { return v * w; }, nullptr);
  // testing/kernels/fusion/softmax.tca, testing/runners/softmax.cu:49-61
  ok &= suite_case("Softmax", 128, 8, 256, 1,
                   [](Builder& b, Expr v, Expr w, std::map<std::string, Expr>&) { return b.Mul(b.Call("expf", {v}), w); }, nullptr, {},
                   [](float v, float w) { return expf(v) * w; }, nullptr);
  // testing/kernels/tiling/transpose.tca
  ok &= suite_case("Transpose", 192, 96, 8, 2, [](Builder& b, Expr v, Expr w, std::map<std::string, Expr>&) { return b.Mul(v, w); }, nullptr, {},
                   [](float v, float w) { return v * w; }, nullptr);
  // testing/kernels/runtime/scale_copy.tca: (gain * v + bias) * w
  ok &= suite_case("ScaleCopy", 512, 512, 4, 2,
                   [](Builder& b, Expr v, Expr w, std::map<std::string, Expr>& sp) {
                     return b.Mul(b.Add(b.Mul(sp["gain"], v), sp["bias"]), w);
                   },
                   nullptr, {{"gain", 1.25f}, {"bias", -0.125f}},
                   [](float v, float w) { return (1.25f * v + -0.125f) * w; }, nullptr);
  // testing/kernels/fusion/axpy3.tca: map | reduce | map
  ok &= suite_case("Axpy3", 512, 512, 4, 2,
                   [](Builder& b, Expr v, Expr w, std::map<std::string, Expr>&) {
                     return b.Add(b.Mul(b.Float32(2.0f), v), b.Mul(b.Float32(0.5f), w));
                   },
                   [](Builder& b, Expr v) { return b.Add(v, b.Mul(b.Float32(0.75f), b.Call("tanhf", {v}))); }, {},
                   [](float v, float w) { return 2.0f * v + 0.5f * w; },
                   [](float v) { return v + 0.75f * tanhf(v); });
  // testing/kernels/llm/layernorm.tca, testing/runners/layernorm.cu:47-58
  ok &= suite_case("Layernorm", 128, 256, 64, 2,
                   [](Builder& b, Expr v, Expr w, std::map<std::string, Expr>&) { return b.Mul(b.Mul(v, v), w); },
                   [](Builder& b, Expr v) {
                     return b.Mul(v, b.Call("rsqrtf", {b.Add(b.Mul(v, b.Float32(1.0f / 64.0f)), b.Float32(1e-5f))}));
                   },
                   {}, [](float v, float w) { return (v * v) * w; },
                   [](float s) { return s * (1.0f / sqrtf(s * (1.0f / 64.0f) + 1e-5f)); });

  {  // internal/e2e/e2e_test.go:228-240: 1024 x 512 row sums -> rank-1 output (the reference's defect D1 shape)
    Builder b("RowSumE2E");
    Dim r = b.Dim("r", 0), c = b.Dim("c", 0);
    Tensor lhs = b.Tensor("lhs", Elem::F32, r, c), out = b.Tensor("out", Elem::F32, r);
    auto ra = b.Stmt().Iter(r, c).Map({At(lhs, r, c)}, [&](Expr v) { return v; });
    auto ar = ra.value.As(r, c).Reduce(b.Float32(0), [&](Expr a, Expr v) { return b.Add(a, v); });
    auto st = ar.value.Store(out, r);
    auto g = b.Build();
    std::vector<float> h(1024 * 512), ref(1024);
    for (unsigned i = 0; i < h.size(); ++i) h[i] = elem(i);
    for (unsigned i = 0; i < 1024; ++i) {
      float acc = 0;
      for (unsigned j = 0; j < 512; ++j) acc += h[i * 512 + j];
      ref[i] = acc;
    }
    ok &= st.ok() && g.ok() &&
          run_and_report("RowSumE2E", g.value, {{"lhs", view(TCAB_F32, {1024, 512})}, {"out", view(TCAB_F32, {1024})}},
                         {h.data(), nullptr}, {}, "out", ref, false);
  }
  {  // pkg/oracle_test.go:17-63 + internal/e2e/frontend_test.go:33-34,194-209: matmul_scale, 64 x 128 x 64, scale 1.5
    const unsigned M = 64, N = 128, Q = 64;
    Builder b("MatmulScale");
    Dim m = b.Dim("m", 0), k = b.Dim("k", 0), n = b.Dim("n", 0);
    Tensor lhs = b.Tensor("lhs", Elem::F32, m, n), rhs = b.Tensor("rhs", Elem::F32, n, k);
    Tensor out = b.Tensor("output", Elem::F32, m, k);
    Expr scale = b.ScalarParam("scale", Elem::F32);
    auto root = b.Stmt().Iter(m, k, n).Map({At(lhs, m, n), At(rhs, n, k)}, [&](Expr l, Expr r) { return b.Mul(l, r); });
    auto ar = root.value.As(m, k, n).Reduce(b.Float32(0.0f), [&](Expr acc, Expr v) { return b.Add(acc, v); });
    auto am = ar.value.Map({}, [&](Expr v) { return b.Mul(v, scale); });
    auto st = am.value.As(m, k).Store(out, m, k);
    auto g = b.Build();
    std::vector<float> hl(M * N), hr(N * Q), ref(M * Q);
    for (unsigned i = 0; i < M * N; ++i) hl[i] = elem(i);
    for (unsigned i = 0; i < N * Q; ++i) hr[i] = elem(i);
    for (unsigned mi = 0; mi < M; ++mi)
      for (unsigned qi = 0; qi < Q; ++qi) {
        float acc = 0.0f;
        for (unsigned ni = 0; ni < N; ++ni) acc += hl[mi * N + ni] * hr[ni * Q + qi];
        ref[mi * Q + qi] = acc * 1.5f;
      }
    ok &= st.ok() && g.ok() &&
          run_and_report("MatmulScale", g.value,
                         {{"lhs", view(TCAB_F32, {M, N})}, {"rhs", view(TCAB_F32, {N, Q})}, {"output", view(TCAB_F32, {M, Q})}},
                         {hl.data(), hr.data(), nullptr}, {{"scale", 1.5f}}, "output", ref, false);
  }
  {  // the bf16 contraction with bias + ReLU, built through the rungs
    const unsigned M = 256, K = 512, N = 256;
    Builder b("GemmBiasRelu");
    Dim m = b.Dim("m", 0), n = b.Dim("n", 0), k = b.Dim("k", 0);
    Tensor A = b.Tensor("a", Elem::BF16, m, k), B = b.Tensor("b", Elem::BF16, k, n);
    Tensor bias = b.Tensor("bias", Elem::F32, n), C = b.Tensor("c", Elem::BF16, m, n);
    auto ra = b.Stmt().Iter(m, n, k).Map({At(A, m, k), At(B, k, n)}, [&](Expr l, Expr r) {
      return b.Mul(b.Cast(l, Elem::F32), b.Cast(r, Elem::F32));
    });
    auto ar = ra.value.As(m, n, k).Reduce(b.Float32(0), [&](Expr a, Expr v) { return b.Add(a, v); });
    auto am = ar.value.Map({At(bias, n)}, [&](Expr v, Expr bb) {
      return b.Cast(b.Call("fmaxf", {b.Add(v, bb), b.Float32(0)}), Elem::BF16);
    });
    auto st = am.value.As(m, n).Store(C, m, n);
    auto g = b.Build();
    std::vector<uint16_t> ha(M * K), hb(K * N);
    std::vector<float> hbias(N), ref(M * N);
    for (unsigned i = 0; i < M * K; ++i) ha[i] = f2bf((elem(i) - 0.5f) * 0.1f);
    for (unsigned i = 0; i < K * N; ++i) hb[i] = f2bf((elem(i + 7u) - 0.5f) * 0.1f);
    for (unsigned i = 0; i < N; ++i) hbias[i] = (elem(i + 3u) - 0.5f) * 0.04f;
    for (unsigned i = 0; i < M; ++i)
      for (unsigned j = 0; j < N; ++j) {
        float acc = 0.0f;
        for (unsigned kk = 0; kk < K; ++kk) acc += bf2f(ha[i * K + kk]) * bf2f(hb[kk * N + j]);
        ref[i * N + j] = bf2f(f2bf(fmaxf(acc + hbias[j], 0.0f)));
      }
    ok &= st.ok() && g.ok() &&
          run_and_report("GemmBiasRelu", g.value,
                         {{"a", view(TCAB_BF16, {M, K})}, {"b", view(TCAB_BF16, {K, N})}, {"bias", view(TCAB_F32, {N})},
                          {"c", view(TCAB_BF16, {M, N})}},
                         {ha.data(), hb.data(), hbias.data(), nullptr}, {}, "c", ref, true);
  }
  return ok;
}

// The same texts the CPU half parses, launched: text -> rungs -> classifier -> C ABI (internal/e2e/frontend_test.go
// takes a .tca through the whole pipeline the same way and compares with a host loop).
static bool tca_gpu_tests() {
  bool ok = true;
  {
    auto r = ParseModule(kTcaWeightedFold);
    const unsigned R = 300, C = 129, K = 8;
    std::vector<float> hx(R * C * K), hz(R * C * K), ref(R * C);
    for (unsigned i = 0; i < hx.size(); ++i) { hx[i] = elem(i); hz[i] = elem(i + 11u); }
    for (unsigned i = 0; i < R * C; ++i) {
      float acc = 0.0f;
      for (unsigned k = 0; k < K; ++k) acc += 2.0f * hx[i * K + k] + -0.5f * hz[i * K + k];
      ref[i] = 0.25f + 0.125f * acc;
    }
    ok &= r.ok() && run_and_report("TcaWeightedFold", r.value[0].graph,
                                   {{"x", view(TCAB_F32, {R, C, K})}, {"z", view(TCAB_F32, {R, C, K})}, {"folded", view(TCAB_F32, {R, C})}},
                                   {hx.data(), hz.data(), nullptr}, {{"w0", 2.0f}, {"w1", -0.5f}, {"lift", 0.125f}}, "folded", ref, false);
  }
  {
    auto r = ParseModule(kTcaMidAxis);
    const unsigned B = 64, K = 6, C = 1000;
    std::vector<float> hx(B * K * C), ref(B * C);
    for (unsigned i = 0; i < hx.size(); ++i) hx[i] = elem(i);
    for (unsigned b = 0; b < B; ++b)
      for (unsigned c = 0; c < C; ++c) {
        float best = -INFINITY;
        for (unsigned k = 0; k < K; ++k) {
          const float v = hx[(b * K + k) * C + c];
          best = fmaxf(best, v * v - 0.5f);
        }
        ref[b * C + c] = best;
      }
    ok &= r.ok() && run_and_report("TcaMidAxisMax", r.value[0].graph, {{"x", view(TCAB_F32, {B, K, C})}, {"m", view(TCAB_F32, {B, C})}},
                                   {hx.data(), nullptr}, {}, "m", ref, false);
  }
  {
    auto r = ParseModule(kTcaScores);
    const unsigned H = 96, N = 200, D = 64;
    std::vector<float> hq(H * D), hk(N * D), ref(H * N);
    for (unsigned i = 0; i < hq.size(); ++i) hq[i] = elem(i);
    for (unsigned i = 0; i < hk.size(); ++i) hk[i] = elem(i + 5u);
    for (unsigned h = 0; h < H; ++h)
      for (unsigned n = 0; n < N; ++n) {
        float acc = 0.0f;
        for (unsigned d = 0; d < D; ++d) acc += hq[h * D + d] * hk[n * D + d];
        ref[h * N + n] = acc * 0.125f;
      }
    ok &= r.ok() && run_and_report("TcaScores", r.value[0].graph,
                                   {{"q", view(TCAB_F32, {H, D})}, {"keys", view(TCAB_F32, {N, D})}, {"s", view(TCAB_F32, {H, N})}},
                                   {hq.data(), hk.data(), nullptr}, {{"temp", 0.125f}}, "s", ref, false);
  }
  {  // a constant extent is checked against the bound tensor at launch
    auto r = ParseModule(kTcaMidAxis);
    DeviceBuf a, o;
    if (cudaMalloc(&a.p, 4 * 5 * 8 * 4) != cudaSuccess || cudaMalloc(&o.p, 4 * 8 * 4) != cudaSuccess) return false;
    Bindings bind;
    tcab_tensor tx = view(TCAB_F32, {4, 5, 8}), tm = view(TCAB_F32, {4, 8});
    tx.data = a.p;
    tm.data = o.p;
    bind.tensors["x"] = tx;
    bind.tensors["m"] = tm;
    const int rc = r.ok() ? Launch(r.value[0].graph, bind, nullptr) : -1;
    std::printf("TCA_CONST_EXTENT %s\n", rc == TCAB_ERR_SHAPE ? "rejected" : "accepted");
    ok &= rc == TCAB_ERR_SHAPE;
  }
  return ok;
}
#endif  // HOST_TESTS_WITH_CUDA

// The k ranges of a middle-axis reduction split over CTAs (the launcher's plan, pure arithmetic): for every
// reduced extent, tile count and occupancy the ranges must tile [0, nk) exactly -- none empty, none
// starting at or past nk -- because a CTA folds rows kbeg..kend of its range without another bound.
static void test_outer_split_plan_covers_k() {
  const int sms = 148;
  const unsigned tiles_list[] = {1, 2, 3, 5, 8, 16, 37, 64, 100, 147};
  unsigned long long bad = 0, split_cases = 0;
  auto one = [&](unsigned long long tiles, unsigned long long cells, unsigned nk, unsigned long long resident, int forced) {
    uint32_t ranges = 0, klen = 0;
    if (tcab_plan_outer_split(tiles, cells, nk, resident, sms, forced, &ranges, &klen) != TCAB_OK) { ++bad; return; }
    if (ranges < 1) { ++bad; return; }
    if (ranges == 1) { if (klen != nk) ++bad; return; }
    ++split_cases;
    const unsigned long long last_beg = static_cast<unsigned long long>(ranges - 1) * klen;
    if (klen == 0 || last_beg >= nk || static_cast<unsigned long long>(ranges) * klen < nk) ++bad;
    if (cells * ranges > 262144ull) ++bad;  // the partials fit the library's scratch
  };
  for (int occ = 1; occ <= 8; ++occ)
    for (unsigned tiles : tiles_list) {
      const unsigned long long resident = static_cast<unsigned long long>(occ) * sms;
      for (unsigned nk = 1; nk <= 300000; ++nk) one(tiles, tiles * 64ull, nk, resident, 0);
      for (unsigned nk = 300007; nk <= 2000000; nk += 997) one(tiles, tiles * 128ull, nk, resident, 0);
    }
  // the shape that exposed an empty trailing range: [1, 66305, 64] with 259 wanted ranges
  one(1, 64, 66305, 259, 0);
  for (int forced : {2, 3, 7, 64, 259, 1000})
    for (unsigned nk = 1; nk <= 70000; ++nk) one(1, 64, nk, 8 * sms, forced);
  CHECK(bad == 0);
  CHECK(split_cases > 100000);
  std::printf("outer split plan: %llu split cases swept, %llu bad\n", split_cases, bad);
}

// pkg/local_test.go:17-68 TestBuilderLocal: a reduction stores into a rank-1 local with a dynamic extent, a
// later statement maps over it; :70-96: a rank >= 2 local with dynamic extents is a recorded declaration error.
static void test_locals_and_typed_expressions() {
  {
    Builder b("local");
    Dim m = b.Dim("m", 0), n = b.Dim("n", 0);
    Tensor lhs = b.Tensor("lhs", Elem::F32, m, n), out = b.Tensor("out", Elem::F32, m);
    Tensor tmp = b.Local("tmp", Elem::F32, {m});
    auto root = b.Stmt().Iter(m, n).Map({At(lhs, m, n)}, [](Expr v) { return v; });
    CHECK(root.ok());
    auto ar = root.value.As(m, n).Reduce(b.Float32(0), [&](Expr acc, Expr v) { return b.Add(acc, v); });
    CHECK(ar.ok());
    CHECK(ar.value.Store(tmp, m).ok());
    auto root2 = b.Stmt().Iter(m, n).Map({At(lhs, m, n), At(tmp, m)}, [&](Expr v, Expr t) { return b.Sub(v, t); });
    CHECK(root2.ok());
    auto ar2 = root2.value.As(m, n).Reduce(b.Float32(0), [&](Expr acc, Expr v) { return b.Add(acc, v); });
    CHECK(ar2.ok());
    auto am = ar2.value.Map({}, [&](Expr v) { return b.Mul(v, b.Float32(2)); });
    CHECK(am.ok());
    CHECK(am.value.As(m).Store(out, m).ok());
    auto g = b.Build();
    CHECK(g.ok());
    CHECK(g.value.statements.size() == 2 && g.value.tensors[2].local);
    auto plans = PlanGraph(g.value);
    CHECK(plans.ok() && plans.value.size() == 2);
    CHECK(plans.ok() && plans.value[1].indexing == std::vector<int>({0, 1}));   // tmp[m] inside (m, n): one value per row
    CHECK(plans.ok() && plans.value[1].map_expr == "(p0 - p1)" && plans.value[1].post_expr == "(p0 * 2.0f)");
  }
  {
    Builder b("local-dyn");
    Dim m = b.Dim("m", 0), n = b.Dim("n", 0);
    b.Tensor("lhs", Elem::F32, m, n);
    b.Local("tmp", Elem::F32, {m, n});
    auto g = b.Build();
    CHECK(!g.ok() && contains(g.err, "a multiplicative GMEM size is not constructed"));
  }
  {
    // pkg/expr.go:137-176, 185-203, 271: operand classes of the whole vocabulary
    Builder b("typed");
    Expr f = b.Float32(1), i = b.Int32(1), u = b.UInt32(1), t = b.Bool(true);
    CHECK(b.Mod(i, i).ok() && contains(b.Mod(f, f).err, "same integer type"));
    CHECK(b.Lt(f, f).typ == Elem::Bool && contains(b.Lt(f, i).err, "operand types differ"));
    CHECK(b.And(t, b.Ge(u, u)).ok() && contains(b.And(f, f).err, "must be bool"));
    CHECK(b.Shl(u, u).ok() && b.BitXor(i, i).ok() && contains(b.BitOr(f, f).err, "same integer type"));
    CHECK(b.Not(t).ok() && contains(b.Not(i).err, "must be bool") && b.BitsNot(i).ok() && contains(b.BitsNot(f).err, "integer type"));
    CHECK(b.Select(t, f, f).typ == Elem::F32);
    CHECK(contains(b.Select(f, f, f).err, "condition must be bool") && contains(b.Select(t, f, i).err, "identical types"));
    CHECK(contains(b.Cast(f, Elem::F32).err, "redundant cast") && contains(b.Cast(t, Elem::F32).err, "arithmetic-to-arithmetic only"));
    std::vector<std::string> caps;
    CHECK(PrintLambda(b.Select(b.Gt(f, b.Float32(0)), f, b.Float32(0)), &caps) == "((1.0f > 0.0f) ? 1.0f : 0.0f)");
    CHECK(PrintLambda(b.Cast(b.BitAnd(b.Shr(u, b.UInt32(3)), b.UInt32(7)), Elem::F32), &caps) == "static_cast<float>(((1u >> 3u) & 7u))");
  }
  {
    // the one added rung (pkg_ext.h): a map stored without a reduction; it keeps every live axis, in order
    Builder b("mapstore");
    Dim m = b.Dim("m", 0), n = b.Dim("n", 0);
    Tensor x = b.Tensor("x", Elem::F32, m, n), bias = b.Tensor("bias", Elem::F32, n), y = b.Tensor("y", Elem::BF16, m, n);
    Tensor z = b.Tensor("z", Elem::F32, m);
    auto root = b.Stmt().Iter(m, n).Map({At(x, m, n), At(bias, n)}, [&](Expr v, Expr c) {
      return b.Cast(b.Call("fmaxf", {b.Add(v, c), b.Float32(0)}), Elem::BF16);
    });
    CHECK(root.ok());
    CHECK(ext::StoreMap(root.value.As(m, n), y, {m, n}).ok());
    auto root2 = b.Stmt().Iter(m, n).Map({At(x, m, n)}, [](Expr v) { return v; });
    auto bad = ext::StoreMap(root2.value.As(m, n), z, {m});
    CHECK(!bad.ok() && contains(bad.err, "a map cannot drop an axis"));
  }
}

int main(int argc, char** argv) {
  test_outer_split_plan_covers_k();
  test_locals_and_typed_expressions();
  test_matmul_scale_builds();
  test_eager_checks();
  test_typestate_and_classification();
  test_tca_frontend();
  std::printf("%d checks, %d failures\n", g_checks, g_failures);
  bool gpu_ok = true;
  if (argc > 1 && std::strcmp(argv[1], "--gpu") == 0) {
#ifdef HOST_TESTS_WITH_CUDA
    gpu_ok = gpu_tests();
    gpu_ok = tca_gpu_tests() && gpu_ok;
    std::printf("GPU_TESTS %s\n", gpu_ok ? "ran" : "incomplete");
#else
    std::printf("GPU_TESTS unavailable: built without CUDA\n");
    gpu_ok = false;
#endif
  }
  return (g_failures == 0 && gpu_ok) ? 0 : 1;
}
