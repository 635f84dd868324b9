// pkg_launch.cpp -- from a built graph to kernel launches: print the lambdas, match each
// statement to an operator class of the kernel library, check the bound tensors the way the
// reference's generated launcher does (internal/cg/cxx/launch.go:23-156: every dim is derived from
// its first tensor occurrence and every other occurrence must agree), call the C ABI.
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
  // fp32 contraction: lhs[m,k] with rhs[k,n] or rhs[n,k], as (m, n, k), out[m,n], piped map without operands
  if (st.operands.size() == 2 && st.reduces.size() == 1 && st.as.size() == 3 && st.iters.size() == 3 &&
      st.operands[0].t.elem == Elem::F32 && st.operands[1].t.elem == Elem::F32 && st.operands[0].axes.size() == 2 &&
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

  // fp32 map | reduce | [map] over identically indexed operands
  p.kind = Plan::ChainReduce;
  if (st.reduces.size() != 1) {
    r.err = "classify: " + std::to_string(st.reduces.size()) +
            " reductions in one chain; the kernel library reduces one axis per launch";
    return r;
  }
  if (st.operands.empty()) {
    r.err = "classify: a map without tensor operands has no kernel class";
    return r;
  }
  const std::vector<Dim>& axes = st.operands[0].axes;
  for (const Operand& op : st.operands) {
    if (op.t.elem != Elem::F32) {
      r.err = "classify: operand " + op.t.name + " is " + ElemName(op.t.elem) +
              "; the chain class is fp32 (bf16 operands are covered by the contraction and layer-norm classes)";
      return r;
    }
    if (!same_axes(op.axes, axes)) {
      r.err = "classify: operand " + op.t.name + " is not indexed like " + st.operands[0].t.name +
              "; operands with different index sets (contractions, broadcasts) need the contraction class, "
              "which this chain does not match";
      return r;
    }
  }
  if (axes.size() != st.iters.size()) {
    r.err = "classify: the operands do not carry every iteration axis";
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
  if (st.out.elem != Elem::F32 || st.elem != Elem::F32) {
    r.err = "classify: the chain class stores fp32";
    return r;
  }
  if (st.has_post && !st.post_operands.empty()) {
    r.err = "classify: a piped map with tensor operands is only covered by the contraction class";
    return r;
  }
  const auto& rd = st.reduces[0];
  if (!rd.init.node || rd.init.node->kind != Node::Const) {
    r.err = "classify: the reduction's init must be a literal";
    return r;
  }
  p.init = static_cast<float>(rd.init.node->value);
  p.reduce_axis = static_cast<uint32_t>(pos);
  std::string err;
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

const std::string& LastError() { return g_last_error; }

namespace {

int elem_dtype(Elem e) {
  switch (e) {
    case Elem::F32: return TCAB_F32;
    case Elem::BF16: return TCAB_BF16;
    case Elem::I32: return TCAB_I32;
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

}  // namespace

int Launch(const Graph& g, const Bindings& bind, void* stream) {
  g_last_error.clear();
  std::map<std::string, uint32_t> extents;  // dim name -> extent from its first tensor occurrence
  for (const Statement& st : g.statements) {
    const Result<Plan> plan = Classify(st);
    if (!plan.ok()) return fail(TCAB_ERR_UNSUPPORTED, plan.err);
    const Plan& p = plan.value;
    if (p.kind == Plan::GemmBiasAct) {
      tcab_tensor a, b, c, bias;
      int rc = bind_tensor(*find_tensor(g, p.a), bind, &extents, &a);
      if (rc == TCAB_OK) rc = bind_tensor(*find_tensor(g, p.b), bind, &extents, &b);
      if (rc == TCAB_OK && !p.bias.empty()) rc = bind_tensor(*find_tensor(g, p.bias), bind, &extents, &bias);
      if (rc == TCAB_OK) rc = bind_tensor(*find_tensor(g, p.out), bind, &extents, &c);
      if (rc != TCAB_OK) return rc;
      rc = tcab_gemm_bias_act(&a, &b, p.bias.empty() ? nullptr : &bias, p.act, &c, stream);
      if (rc != TCAB_OK) return fail(rc, tcab_last_error());
      continue;
    }
    tcab_tensor ins[TCAB_MAX_INPUTS];
    if (p.inputs.size() > TCAB_MAX_INPUTS)
      return fail(TCAB_ERR_UNSUPPORTED, "launch: more than " + std::to_string(TCAB_MAX_INPUTS) + " operands");
    for (size_t i = 0; i < p.inputs.size(); ++i) {
      const int rc = bind_tensor(*find_tensor(g, p.inputs[i]), bind, &extents, &ins[i]);
      if (rc != TCAB_OK) return rc;
    }
    tcab_tensor out;
    int rc = bind_tensor(*find_tensor(g, p.out), bind, &extents, &out);
    if (rc != TCAB_OK) return rc;
    tcab_chain ch;
    std::memset(&ch, 0, sizeof(ch));
    ch.map_expr = p.map_expr.c_str();
    ch.combine_expr = p.combine_expr.c_str();
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
    else
      rc = tcab_chain_reduce(&ch, ins, static_cast<uint32_t>(p.inputs.size()), p.reduce_axis, &out, stream);
    if (rc != TCAB_OK) return fail(rc, tcab_last_error());
  }
  return TCAB_OK;
}

}  // namespace pkg
}  // namespace tcab
