// pkg_launch.cpp -- from a built graph to kernel launches: print the lambdas, match each
// statement to an operator class of the kernel library, check the bound tensors the way the
// reference's generated launcher does (internal/cg/cxx/launch.go:23-156: every dim is derived from
// its first tensor occurrence and every other occurrence must agree), call the C ABI.
#include <cmath>
#include <cstdio>
#include <cstring>

#include "pkg.h"

namespace tcab {
namespace pkg {

namespace {

thread_local std::string g_last_error;

int fail(int status, const std::string& msg) {
  g_last_error = msg;
  return status;
}

std::string print_node(const Node& n, std::vector<std::string>* captures, std::string* err) {
  switch (n.kind) {
    case Node::Const: {
      char buf[64];
      if (n.typ == Elem::F32) {
        if (!(n.value - n.value == 0.0)) {  // inf or nan
          *err = "a non-finite literal has no C spelling in a lambda; pass it as a scalar parameter";
          return "";
        }
        std::snprintf(buf, sizeof(buf), "%.9g", n.value);
        std::string s(buf);
        if (s.find_first_of(".e") == std::string::npos) s += ".0";
        return s + "f";
      }
      if (n.typ == Elem::Bool) return n.value != 0 ? "true" : "false";
      if (n.typ == Elem::U32) {
        std::snprintf(buf, sizeof(buf), "%lluu", static_cast<unsigned long long>(n.value));
        return buf;
      }
      if (n.value < 0) {  // a literal carries no sign (pkg/expr.go: unary minus is a separate operator)
        std::snprintf(buf, sizeof(buf), "(-%lld)", -static_cast<long long>(n.value));
        return buf;
      }
      std::snprintf(buf, sizeof(buf), "%lld", static_cast<long long>(n.value));
      return buf;
    }
    case Node::Param:
      return "p" + std::to_string(n.index);
    case Node::Scalar: {
      for (size_t i = 0; i < captures->size(); ++i)
        if ((*captures)[i] == n.name) return "c" + std::to_string(i);
      captures->push_back(n.name);
      return "c" + std::to_string(captures->size() - 1);
    }
    case Node::Unary:
      return "(" + n.name + print_node(*n.args[0], captures, err) + ")";
    case Node::Binary: {
      // left before right, in separate statements: capture slots are numbered in print order
      const std::string l = print_node(*n.args[0], captures, err);
      const std::string r = print_node(*n.args[1], captures, err);
      return "(" + l + " " + n.name + " " + r + ")";
    }
    case Node::Call: {
      std::string s = n.name + "(";
      for (size_t i = 0; i < n.args.size(); ++i) {
        const std::string a = print_node(*n.args[i], captures, err);
        s += (i ? ", " : "") + a;
      }
      return s + ")";
    }
    case Node::Cast: {  // internal/cg/cxx/expr.go:57-66: static_cast<T>(x), T spelled as internal/cg/cxx/naming.go:21-46
      const char* ts = n.typ == Elem::F32 ? "float" : n.typ == Elem::BF16 ? "__nv_bfloat16" : n.typ == Elem::I32 ? "int32_t"
                       : n.typ == Elem::U32 ? "uint32_t" : nullptr;
      if (ts == nullptr) {
        *err = std::string("a cast to ") + ElemName(n.typ) + " has no kernel in this library (f32, bf16, i32, u32)";
        return "";
      }
      return std::string("static_cast<") + ts + ">(" + print_node(*n.args[0], captures, err) + ")";
    }
    case Node::Select: {  // internal/cg/cxx/expr.go:38-56
      const std::string c = print_node(*n.args[0], captures, err);
      const std::string a = print_node(*n.args[1], captures, err);
      const std::string b = print_node(*n.args[2], captures, err);
      return "(" + c + " ? " + a + " : " + b + ")";
    }
  }
  return "";
}

bool is_param(const std::shared_ptr<Node>& n, int index) { return n && n->kind == Node::Param && n->index == index; }
bool is_const(const std::shared_ptr<Node>& n, double v) { return n && n->kind == Node::Const && n->value == v; }
bool is_binary(const std::shared_ptr<Node>& n, const char* op) {
  return n && n->kind == Node::Binary && n->name == op;
}
bool is_cast_of_param(const std::shared_ptr<Node>& n, Elem to, int index) {
  return n && n->kind == Node::Cast && n->typ == to && is_param(n->args[0], index);
}
// x + y with {x, y} = {param i, param j}
bool is_sum_of_params(const std::shared_ptr<Node>& n, int i, int j) {
  return is_binary(n, "+") && ((is_param(n->args[0], i) && is_param(n->args[1], j)) ||
                               (is_param(n->args[0], j) && is_param(n->args[1], i)));
}
bool same_axes(const std::vector<Dim>& a, const std::vector<Dim>& b) {
  if (a.size() != b.size()) return false;
  for (size_t i = 0; i < a.size(); ++i)
    if (a[i].name != b[i].name) return false;
  return true;
}

// bf16 [m,k] x bf16 [k,n], products in fp32, '+' reducer from 0, optional bias[n] and ReLU, cast to bf16.
bool match_gemm(const Statement& st, Plan* p) {
  if (st.operands.size() != 2 || st.reduces.size() != 1 || st.iters.size() != 3 || st.as.size() != 3) return false;
  const Operand &l = st.operands[0], &r = st.operands[1];
  if (l.t.elem != Elem::BF16 || r.t.elem != Elem::BF16 || l.axes.size() != 2 || r.axes.size() != 2) return false;
  const std::string m = st.as[0].name, n = st.as[1].name, k = st.as[2].name;
  if (l.axes[0].name != m || l.axes[1].name != k || r.axes[0].name != k || r.axes[1].name != n) return false;
  const auto& mb = st.map_body.node;
  if (!is_binary(mb, "*")) return false;
  const bool ab = is_cast_of_param(mb->args[0], Elem::F32, 0) && is_cast_of_param(mb->args[1], Elem::F32, 1);
  const bool ba = is_cast_of_param(mb->args[0], Elem::F32, 1) && is_cast_of_param(mb->args[1], Elem::F32, 0);
  if (!ab && !ba) return false;
  const auto& red = st.reduces[0];
  if (!is_const(red.init.node, 0.0) || !is_sum_of_params(red.body.node, 0, 1)) return false;
  if (!st.has_post || st.out.elem != Elem::BF16 || st.out_axes.size() != 2 || st.out_axes[0].name != m ||
      st.out_axes[1].name != n)
    return false;
  const auto& pb = st.post_body.node;
  if (!pb || pb->kind != Node::Cast || pb->typ != Elem::BF16) return false;
  std::shared_ptr<Node> v = pb->args[0];
  p->act = TCAB_ACT_NONE;
  if (v->kind == Node::Call && v->name == "fmaxf" &&
      (is_const(v->args[1], 0.0) || is_const(v->args[0], 0.0))) {  // fmaxf(x, 0): ReLU
    p->act = TCAB_ACT_RELU;
    v = is_const(v->args[1], 0.0) ? v->args[0] : v->args[1];
  }
  if (st.post_operands.empty()) {
    if (!is_param(v, 0)) return false;
  } else {
    if (st.post_operands.size() != 1) return false;
    const Operand& bo = st.post_operands[0];
    if (bo.t.elem != Elem::F32 || bo.axes.size() != 1 || bo.axes[0].name != n) return false;
    if (!is_sum_of_params(v, 0, 1)) return false;
    p->bias = bo.t.name;
  }
  p->kind = Plan::GemmBiasAct;
  p->a = l.t.name;
  p->b = r.t.name;
  p->out = st.out.name;
  return true;
}

}  // namespace

std::string PrintLambda(const Expr& body, std::vector<std::string>* captures) {
  std::string err;
  const std::string s = body.node ? print_node(*body.node, captures, &err) : "";
  return err.empty() ? s : "";
}

Result<Plan> Classify(const Statement& st) {
  Result<Plan> r;
  if (match_gemm(st, &r.value)) return r;

  Plan& p = r.value;
  // contraction with f32 arithmetic: lhs[m,k] with rhs[k,n] or rhs[n,k], as (m, n, k), out[m,n], piped map without
  // operands; the operands may be f32, bf16, i32 or u32 (the lambda converts explicitly)
  auto movable = [](Elem e) { return e == Elem::F32 || e == Elem::BF16 || e == Elem::I32 || e == Elem::U32; };
  if (st.operands.size() == 2 && st.reduces.size() == 1 && st.as.size() == 3 && st.iters.size() == 3 &&
      movable(st.operands[0].t.elem) && movable(st.operands[1].t.elem) && st.operands[0].axes.size() == 2 &&
      st.operands[1].axes.size() == 2 && st.out.elem == Elem::F32 && st.elem == Elem::F32 &&
      (!st.has_post || st.post_operands.empty())) {
    const std::string m = st.as[0].name, n = st.as[1].name, k = st.as[2].name;
    const auto& la = st.operands[0].axes;
    const auto& ra = st.operands[1].axes;
    const bool kn = ra[0].name == k && ra[1].name == n, nk = ra[0].name == n && ra[1].name == k;
    if (la[0].name == m && la[1].name == k && (kn || nk) && st.out_axes.size() == 2 && st.out_axes[0].name == m &&
        st.out_axes[1].name == n && st.reduces[0].init.node && st.reduces[0].init.node->kind == Node::Const) {
      p.kind = Plan::ChainContract;
      p.rhs_is_nk = nk;
      p.init = static_cast<float>(st.reduces[0].init.node->value);
      std::string err;
      std::vector<std::string> none;
      p.map_expr = print_node(*st.map_body.node, &p.capture_names, &err);
      if (err.empty()) p.combine_expr = print_node(*st.reduces[0].body.node, &none, &err);
      if (err.empty() && !none.empty()) err = "a combiner may not capture scalar parameters";
      if (err.empty() && st.has_post) p.post_expr = print_node(*st.post_body.node, &p.capture_names, &err);
      if (!err.empty()) {
        r.err = "classify: " + err;
        return r;
      }
      p.inputs = {st.operands[0].t.name, st.operands[1].t.name};
      p.out = st.out.name;
      return r;
    }
  }

  // map | reduce | [map], or a map alone (the added rung of pkg_ext.h), over operands that are indexed by every
  // iteration axis, by all but the innermost (one value per row), by the innermost only (one shared row) or, when
  // an axis other than the innermost is reduced, by all but the reduced one (one value per output cell)
  const bool map_only = st.reduces.empty();
  p.kind = map_only ? Plan::Map : Plan::ChainReduce;
  if (st.reduces.size() > 1) {
    r.err = "classify: " + std::to_string(st.reduces.size()) +
            " reductions in one chain; the kernel library reduces one axis per launch";
    return r;
  }
  if (st.operands.empty()) {
    r.err = "classify: a map without tensor operands has no kernel class";
    return r;
  }
  // the operand with every iteration axis fixes the order of the axes in memory
  const Operand* full = nullptr;
  for (const Operand& op : st.operands)
    if (op.axes.size() == st.iters.size() && full == nullptr) full = &op;
  if (full == nullptr) {
    r.err = "classify: no operand carries every iteration axis; a chain needs one operand that fixes the layout";
    return r;
  }
  const std::vector<Dim>& axes = full->axes;
  std::vector<Dim> row_axes(axes.begin(), axes.end() - 1);       // all but the innermost
  std::vector<Dim> col_axes(axes.end() - 1, axes.end());          // the innermost only
  std::vector<Dim> cell_axes;                                     // all but a reduced axis that is not the innermost
  if (!map_only && !st.as.empty()) {
    for (const Dim& d : axes)
      if (d.name != st.as.back().name) cell_axes.push_back(d);
    if (cell_axes.size() == axes.size() || axes.back().name == st.as.back().name) cell_axes.clear();
  }
  for (const Operand& op : st.operands) {
    if (op.t.elem != Elem::F32 && op.t.elem != Elem::BF16 && op.t.elem != Elem::I32 && op.t.elem != Elem::U32) {
      r.err = "classify: operand " + op.t.name + " is " + ElemName(op.t.elem) + "; the kernels move f32, bf16, i32 and u32";
      return r;
    }
    int how = -1;
    if (same_axes(op.axes, axes)) how = 0;
    else if (axes.size() > 1 && same_axes(op.axes, row_axes)) how = 1;
    else if (axes.size() > 1 && same_axes(op.axes, col_axes)) how = 2;
    if (!cell_axes.empty()) how = same_axes(op.axes, axes) ? 0 : same_axes(op.axes, cell_axes) ? 3 : -1;
    if (how < 0) {
      r.err = "classify: operand " + op.t.name + " is not indexed like " + full->t.name +
              ", nor by all but its innermost axis, nor by its innermost axis alone, nor (under a reduction of another "
              "axis) by all but the reduced axis; operands with other index sets "
              "(contractions, transposes) need the contraction class, which this chain does not match";
      return r;
    }
    p.indexing.push_back(how);
  }
  if (st.has_post && !st.post_operands.empty()) {
    r.err = "classify: a piped map with tensor operands is only covered by the contraction class";
    return r;
  }
  std::string err;
  if (map_only) {
    if (!same_axes(st.as, axes) || !same_axes(st.out_axes, axes)) {
      r.err = "classify: a stored map keeps the operands' axis order (a transposing store has no kernel class)";
      return r;
    }
    if (st.out.elem != st.elem) {
      r.err = std::string("classify: the map yields ") + ElemName(st.elem) + " but " + st.out.name + " holds " +
              ElemName(st.out.elem) + "; convert explicitly";
      return r;
    }
    p.map_expr = print_node(*st.map_body.node, &p.capture_names, &err);
    if (!err.empty()) {
      r.err = "classify: " + err;
      return r;
    }
    for (const Operand& op : st.operands) p.inputs.push_back(op.t.name);
    p.out = st.out.name;
    return r;
  }
  const std::string red = st.as.back().name;
  int pos = -1;
  std::vector<Dim> rest;
  for (size_t i = 0; i < axes.size(); ++i) {
    if (axes[i].name == red) pos = static_cast<int>(i);
    else rest.push_back(axes[i]);
  }
  std::vector<Dim> as_rest(st.as.begin(), st.as.end() - 1);
  if (pos < 0 || !same_axes(rest, as_rest) || !same_axes(st.out_axes, rest)) {
    r.err = "classify: the output must keep the operands' axis order minus the reduced axis @" + red +
            " (a transposing store has no kernel class)";
    return r;
  }
  p.reduce_axis = static_cast<uint32_t>(pos);
  if (st.out.elem != Elem::F32 || st.elem != Elem::F32) {
    r.err = "classify: the chain class folds and stores fp32 (convert the mapped value with an explicit cast)";
    return r;
  }
  const auto& rd = st.reduces[0];
  if (!rd.init.node || rd.init.node->kind != Node::Const) {
    r.err = "classify: the reduction's init must be a literal";
    return r;
  }
  p.init = static_cast<float>(rd.init.node->value);
  p.map_expr = print_node(*st.map_body.node, &p.capture_names, &err);
  std::vector<std::string> none;
  if (err.empty()) p.combine_expr = print_node(*rd.body.node, &none, &err);
  if (err.empty() && !none.empty()) err = "a combiner may not capture scalar parameters";
  if (err.empty() && st.has_post) p.post_expr = print_node(*st.post_body.node, &p.capture_names, &err);
  if (!err.empty()) {
    r.err = "classify: " + err;
    return r;
  }
  for (const Operand& op : st.operands) p.inputs.push_back(op.t.name);
  p.out = st.out.name;
  return r;
}

// ---- statement groups that spell a whole row chain ----------------------------------------------------------
namespace {

std::string printed(const Expr& e, std::vector<std::string>* caps) {
  std::string err;
  if (!e.node) return "";
  const std::string s = print_node(*e.node, caps, &err);
  return err.empty() ? s : "";
}

// a reduction over the innermost axis of `x` (operand 0, indexed by every axis) into a local with the other axes
bool is_row_reduction(const Statement& st, size_t n_operands, std::string* map, std::string* comb, std::string* post,
                      std::vector<std::string>* caps) {
  if (st.reduces.size() != 1 || st.operands.size() != n_operands || st.operands[0].axes.size() != st.iters.size() ||
      st.iters.size() < 2 || !st.out.local)
    return false;
  const auto& axes = st.operands[0].axes;
  if (st.as.empty() || st.as.back().name != axes.back().name) return false;
  for (size_t i = 1; i < st.operands.size(); ++i) {   // the others: one value per row
    if (st.operands[i].axes.size() + 1 != axes.size()) return false;
    for (size_t d = 0; d < st.operands[i].axes.size(); ++d)
      if (st.operands[i].axes[d].name != axes[d].name) return false;
  }
  if (!st.reduces[0].init.node || st.reduces[0].init.node->kind != Node::Const) return false;
  std::vector<std::string> none;
  *map = printed(st.map_body, caps);
  *comb = printed(st.reduces[0].body, &none);
  *post = st.has_post ? printed(st.post_body, caps) : "";
  return !map->empty() && !comb->empty() && none.empty() && (!st.has_post || (st.post_operands.empty() && !post->empty()));
}

bool used_elsewhere(const Graph& g, const std::string& tensor, size_t from, size_t to) {
  for (size_t i = 0; i < g.statements.size(); ++i) {
    if (i >= from && i < to) continue;
    for (const Operand& op : g.statements[i].operands)
      if (op.t.name == tensor) return true;
    for (const Operand& op : g.statements[i].post_operands)
      if (op.t.name == tensor) return true;
  }
  return false;
}

bool is_sum(const std::string& c) { return c == "(p0 + p1)" || c == "(p1 + p0)"; }
bool is_max(const std::string& c) { return c == "fmaxf(p0, p1)" || c == "fmaxf(p1, p0)"; }

// m = max_j x;  s = sum_j expf(x - m);  y = expf(x - m) / s      (x, y f32, same shape; m, s locals used nowhere else)
bool match_softmax(const Graph& g, size_t at, Plan* p) {
  if (at + 3 > g.statements.size()) return false;
  const Statement &s1 = g.statements[at], &s2 = g.statements[at + 1], &s3 = g.statements[at + 2];
  std::string map, comb, post;
  std::vector<std::string> caps;
  if (!is_row_reduction(s1, 1, &map, &comb, &post, &caps) || map != "p0" || !is_max(comb) || !post.empty()) return false;
  if (!(s1.reduces[0].init.node->value == -__builtin_inf())) return false;
  const Tensor x = s1.operands[0].t, m = s1.out;
  if (x.elem != Elem::F32) return false;
  if (!is_row_reduction(s2, 2, &map, &comb, &post, &caps) || map != "expf((p0 - p1))" || !is_sum(comb) || !post.empty() ||
      s2.reduces[0].init.node->value != 0.0 || s2.operands[0].t.name != x.name || s2.operands[1].t.name != m.name)
    return false;
  const Tensor s = s2.out;
  if (!s3.reduces.empty() || s3.operands.size() != 3 || s3.operands[0].t.name != x.name || s3.operands[1].t.name != m.name ||
      s3.operands[2].t.name != s.name || s3.out.elem != Elem::F32 || s3.out.dims.size() != x.dims.size())
    return false;
  if (printed(s3.map_body, &caps) != "(expf((p0 - p1)) / p2)" || !caps.empty()) return false;
  if (used_elsewhere(g, m.name, at, at + 3) || used_elsewhere(g, s.name, at, at + 3)) return false;
  p->kind = Plan::SoftmaxRows;
  p->inputs = {x.name};
  p->out = s3.out.name;
  p->fused_locals = {m.name, s.name};
  return true;
}

// mean = (sum_j X) * inv_n;  var = (sum_j (X - mean)^2) * inv_n;  y = (X - mean) * rsqrtf(var + eps) * G + B
// with X = x (f32 rows) or f32(x) (bf16 rows), G, B likewise gamma[j], beta[j], y converted back for bf16 rows;
// inv_n and eps are captured scalar parameters. The statistics are f32 locals used nowhere else.
bool match_layernorm(const Graph& g, size_t at, Plan* p) {
  if (at + 3 > g.statements.size()) return false;
  const Statement &s1 = g.statements[at], &s2 = g.statements[at + 1], &s3 = g.statements[at + 2];
  std::string map, comb, post;
  std::vector<std::string> c1, c2, c3;
  if (!is_row_reduction(s1, 1, &map, &comb, &post, &c1)) return false;
  const Tensor x = s1.operands[0].t, mean = s1.out;
  const bool bf = x.elem == Elem::BF16;
  if (x.elem != Elem::F32 && !bf) return false;
  const std::string X = bf ? "static_cast<float>(p0)" : "p0";
  if (map != X || !is_sum(comb) || post != "(p0 * c0)" || c1.size() != 1 || s1.reduces[0].init.node->value != 0.0) return false;
  if (!is_row_reduction(s2, 2, &map, &comb, &post, &c2) || s2.operands[0].t.name != x.name || s2.operands[1].t.name != mean.name ||
      map != "((" + X + " - p1) * (" + X + " - p1))" || !is_sum(comb) || post != "(p0 * c0)" || c2 != c1 ||
      s2.reduces[0].init.node->value != 0.0)
    return false;
  const Tensor var = s2.out;
  if (!s3.reduces.empty() || s3.operands.size() != 5 || s3.operands[0].t.name != x.name || s3.operands[1].t.name != mean.name ||
      s3.operands[2].t.name != var.name || s3.out.elem != x.elem || s3.out.dims.size() != x.dims.size())
    return false;
  const Tensor gamma = s3.operands[3].t, beta = s3.operands[4].t;
  if (gamma.elem != x.elem || beta.elem != x.elem || gamma.dims.size() != 1 || beta.dims.size() != 1) return false;
  const std::string G = bf ? "static_cast<float>(p3)" : "p3", B = bf ? "static_cast<float>(p4)" : "p4";
  const std::string body = "((((" + X + " - p1) * rsqrtf((p2 + c0))) * " + G + ") + " + B + ")";
  if (printed(s3.map_body, &c3) != (bf ? "static_cast<__nv_bfloat16>(" + body + ")" : body) || c3.size() != 1) return false;
  if (used_elsewhere(g, mean.name, at, at + 3) || used_elsewhere(g, var.name, at, at + 3)) return false;
  p->kind = Plan::LayernormRows;
  p->inputs = {x.name, gamma.name, beta.name};
  p->out = s3.out.name;
  p->eps_scalar = c3[0];
  p->capture_names = c1;   // inv_n: checked against the row length at launch
  p->fused_locals = {mean.name, var.name};
  return true;
}

}  // namespace

Result<std::vector<Plan>> PlanGraph(const Graph& g) {
  Result<std::vector<Plan>> r;
  for (size_t i = 0; i < g.statements.size();) {
    Plan fused;
    if (match_softmax(g, i, &fused) || match_layernorm(g, i, &fused)) {
      r.value.push_back(fused);
      i += 3;
      continue;
    }
    const Result<Plan> one = Classify(g.statements[i]);
    if (!one.ok()) {
      r.err = "statement " + std::to_string(i) + " (" + g.statements[i].out.name + "): " + one.err;
      r.value.clear();
      return r;
    }
    r.value.push_back(one.value);
    ++i;
  }
  return r;
}

const std::string& LastError() { return g_last_error; }

namespace {

int elem_dtype(Elem e) {
  switch (e) {
    case Elem::F32: return TCAB_F32;
    case Elem::BF16: return TCAB_BF16;
    case Elem::I32: return TCAB_I32;
    case Elem::U32: return TCAB_U32;
    default: return -1;
  }
}

// The generated launcher's shape contract, by name.
int bind_tensor(const Tensor& t, const Bindings& bind, std::map<std::string, uint32_t>* extents, tcab_tensor* out) {
  auto it = bind.tensors.find(t.name);
  if (it == bind.tensors.end()) return fail(TCAB_ERR_INVALID_ARG, "launch: tensor " + t.name + " is not bound");
  const tcab_tensor& b = it->second;
  if (b.rank != t.dims.size())
    return fail(TCAB_ERR_SHAPE, "launch: " + t.name + " is declared with rank " + std::to_string(t.dims.size()) +
                                    ", bound with rank " + std::to_string(b.rank));
  if (b.dtype != elem_dtype(t.elem))
    return fail(TCAB_ERR_DTYPE, "launch: " + t.name + " is declared " + ElemName(t.elem) + ", bound with another type");
  for (size_t i = 0; i < t.dims.size(); ++i) {
    const Dim& d = t.dims[i];
    if (d.extent > 0 && b.dims[i] != static_cast<uint32_t>(d.extent))
      return fail(TCAB_ERR_SHAPE, "launch: " + t.name + ".Dim(" + std::to_string(i) + ") must equal " +
                                      std::to_string(d.extent) + " (dim " + d.name + ")");
    auto e = extents->find(d.name);
    if (e == extents->end()) {
      (*extents)[d.name] = b.dims[i];
    } else if (e->second != b.dims[i]) {
      return fail(TCAB_ERR_SHAPE, "launch: " + t.name + ".Dim(" + std::to_string(i) + ") must equal " + d.name +
                                      " (dim " + d.name + ")");
    }
  }
  *out = b;
  return TCAB_OK;
}

const Tensor* find_tensor(const Graph& g, const std::string& name) {
  for (const Tensor& t : g.tensors)
    if (t.name == name) return &t;
  return nullptr;
}

// An operand that lacks axes of the iteration is handed to the kernel library with the iteration's rank and
// extent 1 where it has no axis: [rows..., 1] for a value per row, [1..., cols] for a shared row.
tcab_tensor with_unit_axes(const tcab_tensor& t, int how, uint32_t rank, uint32_t reduce_axis) {
  if (how == 0) return t;
  tcab_tensor v = t;
  v.rank = rank;
  for (uint32_t i = 0; i < rank; ++i) v.dims[i] = 1;
  if (how == 1) for (uint32_t i = 0; i < t.rank && i + 1 < rank; ++i) v.dims[i] = t.dims[i];
  if (how == 2) v.dims[rank - 1] = t.dims[t.rank - 1];
  if (how == 3)
    for (uint32_t i = 0, j = 0; i < rank; ++i)
      if (i != reduce_axis && j < t.rank) v.dims[i] = t.dims[j++];
  return v;
}

}  // namespace

int Launch(const Graph& g, const Bindings& bind, void* stream) {
  g_last_error.clear();
  std::map<std::string, uint32_t> extents;  // dim name -> extent from its first tensor occurrence
  const Result<std::vector<Plan>> plans = PlanGraph(g);
  if (!plans.ok()) return fail(TCAB_ERR_UNSUPPORTED, plans.err);
  auto bound = [&](const std::string& name, tcab_tensor* out) {
    const Tensor* t = find_tensor(g, name);
    if (t == nullptr) return fail(TCAB_ERR_INVALID_ARG, "launch: tensor " + name + " is not declared");
    if (t->local && bind.tensors.find(name) == bind.tensors.end())
      return fail(TCAB_ERR_INVALID_ARG, "launch: local " + name + " is not bound: an intermediate between two statements "
                                        "needs device memory of its shape from the caller, like every other tensor");
    return bind_tensor(*t, bind, &extents, out);
  };
  for (const Plan& p : plans.value) {
    if (p.kind == Plan::GemmBiasAct) {
      tcab_tensor a, b, c, bias;
      int rc = bound(p.a, &a);
      if (rc == TCAB_OK) rc = bound(p.b, &b);
      if (rc == TCAB_OK && !p.bias.empty()) rc = bound(p.bias, &bias);
      if (rc == TCAB_OK) rc = bound(p.out, &c);
      if (rc != TCAB_OK) return rc;
      rc = tcab_gemm_bias_act(&a, &b, p.bias.empty() ? nullptr : &bias, p.act, &c, stream);
      if (rc != TCAB_OK) return fail(rc, tcab_last_error());
      continue;
    }
    if (p.kind == Plan::SoftmaxRows) {
      tcab_tensor x, y;
      int rc = bound(p.inputs[0], &x);
      if (rc == TCAB_OK) rc = bound(p.out, &y);
      if (rc != TCAB_OK) return rc;
      rc = tcab_softmax_rows(&x, &y, stream);
      if (rc != TCAB_OK) return fail(rc, tcab_last_error());
      continue;
    }
    if (p.kind == Plan::LayernormRows) {
      tcab_tensor x, gm, bt, y;
      int rc = bound(p.inputs[0], &x);
      if (rc == TCAB_OK) rc = bound(p.inputs[1], &gm);
      if (rc == TCAB_OK) rc = bound(p.inputs[2], &bt);
      if (rc == TCAB_OK) rc = bound(p.out, &y);
      if (rc != TCAB_OK) return rc;
      auto eps = bind.scalars.find(p.eps_scalar);
      auto inv = bind.scalars.find(p.capture_names[0]);
      if (eps == bind.scalars.end()) return fail(TCAB_ERR_INVALID_ARG, "launch: scalar " + p.eps_scalar + " is not bound");
      if (inv == bind.scalars.end()) return fail(TCAB_ERR_INVALID_ARG, "launch: scalar " + p.capture_names[0] + " is not bound");
      // the one-launch operator divides by the row length itself: the captured factor must be its reciprocal
      const float want = 1.0f / static_cast<float>(x.dims[x.rank - 1]);
      if (!(std::fabs(inv->second - want) <= 1e-6f * want))
        return fail(TCAB_ERR_INVALID_ARG, "launch: scalar " + p.capture_names[0] + " must be 1 / (row length) for the mean and "
                                          "variance statements to be a layer-norm");
      rc = tcab_layernorm_rows(&x, &gm, &bt, eps->second, &y, stream);
      if (rc != TCAB_OK) return fail(rc, tcab_last_error());
      continue;
    }
    tcab_tensor ins[TCAB_MAX_INPUTS];
    if (p.inputs.size() > TCAB_MAX_INPUTS)
      return fail(TCAB_ERR_UNSUPPORTED, "launch: more than " + std::to_string(TCAB_MAX_INPUTS) + " operands");
    uint32_t rank = 0;
    for (size_t i = 0; i < p.inputs.size(); ++i) {
      const int rc = bound(p.inputs[i], &ins[i]);
      if (rc != TCAB_OK) return rc;
      if (i < p.indexing.size() && p.indexing[i] == 0 && rank == 0) rank = ins[i].rank;
    }
    for (size_t i = 0; i < p.inputs.size() && i < p.indexing.size(); ++i) ins[i] = with_unit_axes(ins[i], p.indexing[i], rank, p.reduce_axis);
    tcab_tensor out;
    int rc = bound(p.out, &out);
    if (rc != TCAB_OK) return rc;
    tcab_chain ch;
    std::memset(&ch, 0, sizeof(ch));
    ch.map_expr = p.map_expr.c_str();
    ch.combine_expr = p.combine_expr.empty() ? nullptr : p.combine_expr.c_str();
    ch.post_expr = p.post_expr.empty() ? nullptr : p.post_expr.c_str();
    ch.init = p.init;
    if (p.capture_names.size() > TCAB_MAX_CAPTURES)
      return fail(TCAB_ERR_UNSUPPORTED, "launch: more than " + std::to_string(TCAB_MAX_CAPTURES) + " scalar captures");
    ch.n_captures = static_cast<uint32_t>(p.capture_names.size());
    for (size_t i = 0; i < p.capture_names.size(); ++i) {
      auto it = bind.scalars.find(p.capture_names[i]);
      if (it == bind.scalars.end())
        return fail(TCAB_ERR_INVALID_ARG, "launch: scalar " + p.capture_names[i] + " is not bound");
      ch.captures[i] = it->second;
    }
    if (p.kind == Plan::ChainContract)
      rc = tcab_chain_contract(&ch, &ins[0], &ins[1], p.rhs_is_nk ? 1 : 0, &out, stream);
    else if (p.kind == Plan::Map)
      rc = tcab_map(&ch, ins, static_cast<uint32_t>(p.inputs.size()), &out, stream);
    else
      rc = tcab_chain_reduce(&ch, ins, static_cast<uint32_t>(p.inputs.size()), p.reduce_axis, &out, stream);
    if (rc != TCAB_OK) return fail(rc, tcab_last_error());
  }
  return TCAB_OK;
}

}  // namespace pkg
}  // namespace tcab
