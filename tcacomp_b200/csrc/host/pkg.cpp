// pkg.cpp -- the builder rungs and the expression DSL (see pkg.h). The classification and launch
// half lives in pkg_launch.cpp.
#include "pkg_ext.h"

#include <cmath>
#include <set>

namespace tcab {
namespace pkg {

const char* ElemName(Elem e) {
  switch (e) {
    case Elem::F32: return "f32";
    case Elem::BF16: return "bf16";
    case Elem::F16: return "f16";
    case Elem::I32: return "i32";
    case Elem::U32: return "u32";
    case Elem::Bool: return "bool";
  }
  return "?";
}

namespace {
bool is_float(Elem e) { return e == Elem::F32 || e == Elem::BF16 || e == Elem::F16; }
bool is_int(Elem e) { return e == Elem::I32 || e == Elem::U32; }
bool is_arith(Elem e) { return is_float(e) || is_int(e); }
}  // namespace

// The statement chain under construction (pkg/chain.go: type chain).
struct Builder::Chain {
  Builder* b = nullptr;
  Statement st;
  std::vector<pkg::Dim> live;  // live axes at this point of the chain
  Elem elem = Elem::F32;
  std::string deferred;        // first violation of a rung that cannot return an error
  bool stored = false;

  int liveIndex(const std::string& name) const {
    for (size_t i = 0; i < live.size(); ++i)
      if (live[i].name == name) return static_cast<int>(i);
    return -1;
  }
  void deferErr(const std::string& e) {
    if (!e.empty() && deferred.empty()) deferred = e;
  }
  // pkg/chain.go pending(): declaration errors first, then the chain's own deferred error.
  std::string pending() const {
    if (!b->decl_err_.empty()) return b->decl_err_;
    return deferred;
  }
};

Builder::Builder(std::string name) { g_.name = std::move(name); }

void Builder::noteDeclErr(const std::string& e) {
  if (!e.empty() && decl_err_.empty()) decl_err_ = e;
}

std::string Builder::checkDim(const pkg::Dim& d, const std::string& what) const {
  if (d.b != this || dims_.find(d.name) == dims_.end())
    return what + ": dim @\"" + d.name + "\" is not declared in this builder";
  return "";
}

pkg::Dim Builder::Dim(const std::string& name, int extent) {
  if (final_) noteDeclErr("dim " + name + ": builder already finalized by Build");
  if (extent < 0)
    noteDeclErr("dim " + name + ": extent must be >= 0 (0 = dynamic), got " + std::to_string(extent));
  if (dims_.count(name)) noteDeclErr("dim " + name + ": already declared");
  pkg::Dim d;
  d.b = this;
  d.name = name;
  d.extent = extent;
  dims_[name] = d;
  g_.dims.push_back(d);
  return d;
}

pkg::Tensor Builder::Tensor(const std::string& name, Elem elem, const std::vector<pkg::Dim>& dims) {
  if (final_) noteDeclErr("tensor " + name + ": builder already finalized by Build");
  if (tensors_.count(name)) noteDeclErr("tensor " + name + ": already declared");
  for (const pkg::Dim& d : dims) noteDeclErr(checkDim(d, "tensor " + name));
  pkg::Tensor t;
  t.b = this;
  t.name = name;
  t.dims = dims;
  t.elem = elem;
  tensors_[name] = t;
  g_.tensors.push_back(t);
  return t;
}

pkg::Tensor Builder::Local(const std::string& name, Elem elem, const std::vector<pkg::Dim>& dims) {
  if (final_) noteDeclErr("local " + name + ": builder already finalized by Build");
  if (tensors_.count(name)) noteDeclErr("local " + name + ": already declared");
  if (dims.empty()) noteDeclErr("local " + name + ": must be a tensor type");
  bool dynamic = false;
  for (const pkg::Dim& d : dims) {
    noteDeclErr(checkDim(d, "local " + name));
    dynamic = dynamic || d.extent == 0;
  }
  if (dims.size() > 1 && dynamic)
    noteDeclErr("local " + name + ": rank " + std::to_string(dims.size()) +
                " with dynamic extents is not v0 (a multiplicative GMEM size is not constructed)");
  pkg::Tensor t;
  t.b = this;
  t.name = name;
  t.dims = dims;
  t.elem = elem;
  t.local = true;
  tensors_[name] = t;
  g_.tensors.push_back(t);
  return t;
}

Expr Builder::ScalarParam(const std::string& name, Elem elem) {
  if (final_) noteDeclErr("scalar " + name + ": builder already finalized by Build");
  if (scalars_.count(name)) noteDeclErr("scalar " + name + ": already declared");
  scalars_[name] = elem;
  g_.scalars.emplace_back(name, elem);
  auto n = std::make_shared<Node>();
  n->kind = Node::Scalar;
  n->typ = elem;
  n->name = name;
  return Expr{this, n, elem, ""};
}

StmtIter Builder::Stmt() {
  if (final_) noteDeclErr("stmt: builder already finalized by Build");
  chain_ = std::make_shared<Chain>();
  chain_->b = this;
  StmtIter s;
  s.c_ = chain_;
  return s;
}

Result<Graph> Builder::Build() {
  Result<Graph> r;
  if (!decl_err_.empty()) {
    r.err = decl_err_;
    return r;
  }
  if (chain_ && !chain_->stored) {
    r.err = "build: statement chain was never stored";
    return r;
  }
  final_ = true;
  r.value = g_;
  return r;
}

// ---- expressions -----------------------------------------------------------

Expr Builder::bad(const std::string& e) {
  Expr x;
  x.b = this;
  x.err = e;
  return x;
}

// The shared bottom of every binary operator (pkg/expr.go:137-176 typedBinOp): operand errors propagate,
// operands belong to this builder and share one type, the type satisfies the operator's class, comparisons
// yield bool.
Expr Builder::binop(const char* op, Expr x, Expr y, const char* cls) {
  if (!x.ok()) return bad(x.err);
  if (!y.ok()) return bad(y.err);
  if (x.b != this || y.b != this) return bad(std::string(op) + ": operands come from a different builder");
  if (x.typ != y.typ)
    return bad(std::string(op) + ": operand types differ (" + ElemName(x.typ) + " vs " + ElemName(y.typ) +
               "); implicit promotions are not supported (syntax-design.md §4.6 rule 17)");
  Elem result = x.typ;
  const std::string c = cls;
  if (c == "arithmetic") {
    if (!is_arith(x.typ))
      return bad(std::string(op) + ": operands must have the same arithmetic type, got " + ElemName(x.typ));
  } else if (c == "integer") {
    if (!is_int(x.typ)) return bad(std::string(op) + ": operands must have the same integer type, got " + ElemName(x.typ));
  } else if (c == "bool") {
    if (x.typ != Elem::Bool) return bad(std::string(op) + ": operands must be bool, got " + ElemName(x.typ));
  } else {  // comparable: every supported scalar type, result bool
    result = Elem::Bool;
  }
  auto n = std::make_shared<Node>();
  n->kind = Node::Binary;
  n->typ = result;
  n->name = op;
  n->args = {x.node, y.node};
  return Expr{this, n, result, ""};
}

Expr Builder::Add(Expr x, Expr y) { return binop("+", x, y); }
Expr Builder::Sub(Expr x, Expr y) { return binop("-", x, y); }
Expr Builder::Mul(Expr x, Expr y) { return binop("*", x, y); }
Expr Builder::Div(Expr x, Expr y) { return binop("/", x, y); }
Expr Builder::Mod(Expr x, Expr y) { return binop("%", x, y, "integer"); }
Expr Builder::Eq(Expr x, Expr y) { return binop("==", x, y, "comparable"); }
Expr Builder::Ne(Expr x, Expr y) { return binop("!=", x, y, "comparable"); }
Expr Builder::Lt(Expr x, Expr y) { return binop("<", x, y, "comparable"); }
Expr Builder::Le(Expr x, Expr y) { return binop("<=", x, y, "comparable"); }
Expr Builder::Gt(Expr x, Expr y) { return binop(">", x, y, "comparable"); }
Expr Builder::Ge(Expr x, Expr y) { return binop(">=", x, y, "comparable"); }
Expr Builder::And(Expr x, Expr y) { return binop("&&", x, y, "bool"); }
Expr Builder::Or(Expr x, Expr y) { return binop("||", x, y, "bool"); }
Expr Builder::BitAnd(Expr x, Expr y) { return binop("&", x, y, "integer"); }
Expr Builder::BitOr(Expr x, Expr y) { return binop("|", x, y, "integer"); }
Expr Builder::BitXor(Expr x, Expr y) { return binop("^", x, y, "integer"); }
Expr Builder::Shl(Expr x, Expr y) { return binop("<<", x, y, "integer"); }
Expr Builder::Shr(Expr x, Expr y) { return binop(">>", x, y, "integer"); }

// pkg/expr.go typedUnary: Neg / Pos arithmetic, Not bool, BitsNot integer.
Expr Builder::unop(const char* op, Expr x, const char* cls) {
  if (!x.ok()) return bad(x.err);
  if (x.b != this) return bad(std::string(op) + ": operand comes from a different builder");
  const std::string c = cls;
  if (c == "arithmetic" && !is_arith(x.typ))
    return bad(std::string(op) + ": operand must have an arithmetic type, got " + ElemName(x.typ));
  if (c == "integer" && !is_int(x.typ))
    return bad(std::string(op) + ": operand must have an integer type, got " + ElemName(x.typ));
  if (c == "bool" && x.typ != Elem::Bool) return bad(std::string(op) + ": operand must be bool, got " + ElemName(x.typ));
  auto n = std::make_shared<Node>();
  n->kind = Node::Unary;
  n->typ = x.typ;
  n->name = op;
  n->args = {x.node};
  return Expr{this, n, x.typ, ""};
}

Expr Builder::Neg(Expr x) { return unop("-", x, "arithmetic"); }
Expr Builder::Pos(Expr x) { return unop("+", x, "arithmetic"); }
Expr Builder::Not(Expr x) { return unop("!", x, "bool"); }
Expr Builder::BitsNot(Expr x) { return unop("~", x, "integer"); }

Expr Builder::UInt32(uint32_t v) {
  auto n = std::make_shared<Node>();
  n->kind = Node::Const;
  n->typ = Elem::U32;
  n->value = v;
  return Expr{this, n, Elem::U32, ""};
}

Expr Builder::Bool(bool v) {
  auto n = std::make_shared<Node>();
  n->kind = Node::Const;
  n->typ = Elem::Bool;
  n->value = v ? 1 : 0;
  return Expr{this, n, Elem::Bool, ""};
}

// pkg/expr.go:271 Select: the condition must be bool and the branches identically typed.
Expr Builder::Select(Expr cond, Expr a, Expr b) {
  for (const Expr* e : {&cond, &a, &b})
    if (!e->ok()) return bad(e->err);
  if (cond.b != this || a.b != this || b.b != this) return bad("select: operands come from different builders");
  if (cond.typ != Elem::Bool) return bad(std::string("select: condition must be bool, got ") + ElemName(cond.typ));
  if (a.typ != b.typ)
    return bad(std::string("select: branches must have identical types, got ") + ElemName(a.typ) + " vs " + ElemName(b.typ));
  auto n = std::make_shared<Node>();
  n->kind = Node::Select;
  n->typ = a.typ;
  n->args = {cond.node, a.node, b.node};
  return Expr{this, n, a.typ, ""};
}

Expr Builder::Float32(float v) {
  auto n = std::make_shared<Node>();
  n->kind = Node::Const;
  n->typ = Elem::F32;
  n->value = v;
  return Expr{this, n, Elem::F32, ""};
}

Expr Builder::Int32(int32_t v) {
  auto n = std::make_shared<Node>();
  n->kind = Node::Const;
  n->typ = Elem::I32;
  n->value = v;
  return Expr{this, n, Elem::I32, ""};
}

// Casts are arithmetic <-> arithmetic only (internal/ir/types.go:60-62).
Expr Builder::Cast(Expr x, Elem to) {
  if (!x.ok()) return bad(x.err);
  if (x.b != this) return bad("cast: operand comes from a different builder");
  if (x.typ == to) return bad(std::string("cast: redundant cast to ") + ElemName(to));
  if (!is_arith(x.typ) || !is_arith(to))
    return bad(std::string("cast: pair ") + ElemName(x.typ) + " -> " + ElemName(to) +
               " is not in the v0 cast registry (arithmetic-to-arithmetic only)");
  auto n = std::make_shared<Node>();
  n->kind = Node::Cast;
  n->typ = to;
  n->args = {x.node};
  return Expr{this, n, to, ""};
}

// The fp32 builtins, emitted verbatim by the reference (internal/cg/cxx/naming.go:188-198).
Expr Builder::Call(const std::string& builtin, const std::vector<Expr>& args) {
  static const std::map<std::string, size_t> arity = {{"expf", 1}, {"logf", 1},  {"sqrtf", 1}, {"rsqrtf", 1},
                                                      {"fabsf", 1}, {"tanhf", 1}, {"sinf", 1},  {"cosf", 1},
                                                      {"fminf", 2}, {"fmaxf", 2}, {"fmaf", 3}};
  auto it = arity.find(builtin);
  if (it == arity.end()) return bad("call: unknown builtin " + builtin);
  if (args.size() != it->second)
    return bad("call: " + builtin + " takes " + std::to_string(it->second) + " arguments, got " +
               std::to_string(args.size()));
  auto n = std::make_shared<Node>();
  n->kind = Node::Call;
  n->typ = Elem::F32;
  n->name = builtin;
  for (const Expr& a : args) {
    if (!a.ok()) return bad(a.err);
    if (a.b != this) return bad("call: argument comes from a different builder");
    if (a.typ != Elem::F32) return bad("call: " + builtin + " takes f32 arguments, got " + ElemName(a.typ));
    n->args.push_back(a.node);
  }
  return Expr{this, n, Elem::F32, ""};
}

// ---- rungs -----------------------------------------------------------------

namespace {

Expr param(Builder* b, int index, Elem typ) {
  auto n = std::make_shared<Node>();
  n->kind = Node::Param;
  n->typ = typ;
  n->index = index;
  return Expr{b, n, typ, ""};
}

std::string join(const std::vector<std::string>& v) {
  std::string s;
  for (size_t i = 0; i < v.size(); ++i) s += (i ? ", " : "") + v[i];
  return s;
}

}  // namespace

RootMap StmtIter::IterV(const std::vector<Dim>& dims) {
  auto& c = *c_;
  if (dims.empty()) c.deferErr("iter: an iteration cluster needs at least one dim");
  for (const Dim& d : dims) {
    const std::string e = c.b->checkDim(d, "iter");
    if (!e.empty()) {
      c.deferErr(e);
      continue;
    }
    if (c.liveIndex(d.name) >= 0) {
      c.deferErr("iter: dim @" + d.name + " is listed twice");
      continue;
    }
    c.st.iters.push_back(d);
    c.live.push_back(d);
  }
  RootMap r;
  r.c_ = c_;
  return r;
}

// Shared by the root map and the piped map (pkg/chain.go buildMapLambda, checkOperand: structural
// indexing, positional binding, live axes only).
static std::string build_map_lambda(Builder* b, std::shared_ptr<Builder::Chain> cp,
                                    const std::map<std::string, Tensor>& declared, const std::vector<Operand>& ops,
                                    const Lambda& fn, bool piped, Elem piped_elem, Expr* body,
                                    const std::function<int(const std::string&)>& live_index,
                                    const std::function<std::string(const Dim&, const std::string&)>& check_dim) {
  (void)cp;
  if (!fn.call) return "map: nil lambda";
  const int want = static_cast<int>(ops.size()) + (piped ? 1 : 0);
  if (fn.arity >= 0 && fn.arity != want)
    return "map: lambda arity mismatch: the lambda takes " + std::to_string(fn.arity) + " parameters, the map feeds " +
           std::to_string(want) + (piped ? " (the piped value plus the operands)" : " (one per operand)");
  std::vector<Expr> args;
  if (piped) args.push_back(param(b, 0, piped_elem));
  for (const Operand& op : ops) {
    const Tensor& t = op.t;
    auto it = declared.find(t.name);
    if (t.b != b || it == declared.end()) return "map: tensor \"" + t.name + "\" is not declared in this builder";
    if (op.axes.size() != t.dims.size())
      return "map: operand " + t.name + " has " + std::to_string(op.axes.size()) + " subscripts for rank " +
             std::to_string(t.dims.size()) + " (structural indexing, syntax-design.md §4.4 rule 9)";
    for (size_t i = 0; i < op.axes.size(); ++i) {
      const std::string e = check_dim(op.axes[i], "map operand " + t.name);
      if (!e.empty()) return e;
      if (op.axes[i].name != t.dims[i].name)
        return "map: operand " + t.name + " subscript " + std::to_string(i) + " binds @" + op.axes[i].name +
               ", but dim " + std::to_string(i) + " of " + t.name + " is @" + t.dims[i].name +
               " (structural indexing binds subscripts positionally)";
      if (live_index(op.axes[i].name) < 0)
        return "map: operand " + t.name + " binds @" + op.axes[i].name +
               ", which is not a live axis at this point of the chain";
    }
    args.push_back(param(b, static_cast<int>(args.size()), t.elem));
  }
  *body = fn.call(args);
  if (!body->ok()) return body->err;
  if (body->b != b) return "map: lambda body comes from a different builder";
  return "";
}

Result<RootAs> RootMap::Map(const std::vector<Operand>& ops, Lambda fn) {
  auto& c = *c_;
  Result<RootAs> r;
  r.err = c.pending();
  if (!r.ok()) return r;
  if (c.st.iters.empty()) {
    r.err = "map: the iteration cluster is empty";
    return r;
  }
  Builder* b = c.b;
  Expr body;
  r.err = build_map_lambda(
      b, c_, b->tensors_, ops, fn, false, Elem::F32, &body, [&](const std::string& n) { return c.liveIndex(n); },
      [&](const Dim& d, const std::string& w) { return b->checkDim(d, w); });
  if (!r.ok()) return r;
  c.st.operands = ops;
  c.st.map_body = body;
  r.value.c_ = c_;
  return r;
}

MidChain RootAs::AsV(const std::vector<Dim>& dims) {
  auto& c = *c_;
  if (c.pending().empty()) {
    // pkg/chain.go checkAsPermutation: every iteration axis exactly once
    std::string e;
    if (dims.size() != c.st.iters.size()) {
      e = "root map: as lists " + std::to_string(dims.size()) + " axes, the iteration cluster has " +
          std::to_string(c.st.iters.size());
    } else {
      std::set<std::string> seen;
      std::vector<std::string> dups, missing;
      for (const Dim& d : dims) {
        const std::string ce = c.b->checkDim(d, "root map as");
        if (!ce.empty() && e.empty()) e = ce;
        if (seen.count(d.name)) dups.push_back("@" + d.name);
        seen.insert(d.name);
      }
      for (const Dim& it : c.st.iters)
        if (!seen.count(it.name)) missing.push_back("@" + it.name);
      if (e.empty() && (!dups.empty() || !missing.empty()))
        e = "root map: as must list every live axis exactly once; duplicated: " + join(dups) +
            "; missing: " + join(missing);
    }
    c.deferErr(e);
  }
  c.st.as = dims;
  c.elem = c.st.map_body.typ;
  c.live = dims;
  MidChain m;
  m.c_ = c_;
  return m;
}

// pkg/chain.go buildReduce: homogeneous reducer, removes the LAST live axis.
static std::string build_reduce(Builder::Chain& c, Builder* b, Expr init, const Combiner& fn) {
  if (!fn) return "reduce: nil combiner";
  if (!init.ok()) return init.err;
  if (init.b != b) return "reduce: init comes from a different builder";
  if (c.live.empty()) return "reduce: no live axis left to reduce";
  const Elem T = c.elem;
  if (init.typ != T)
    return std::string("reduce: homogeneous reducer violated (tca.md §4.2): init has type ") + ElemName(init.typ) +
           ", the piped value has element type " + ElemName(T);
  const Expr body = fn(param(b, 0, T), param(b, 1, T));
  if (!body.ok()) return body.err;
  if (body.b != b) return "reduce: combiner body comes from a different builder";
  if (body.typ != T)
    return std::string("reduce: homogeneous reducer violated (tca.md §4.2): combiner returns ") +
           ElemName(body.typ) + ", want " + ElemName(T);
  c.st.reduces.push_back(Statement::Reduce{init, body});
  c.live.pop_back();
  return "";
}

Result<AfterReduce> MidChain::Reduce(Expr init, Combiner fn) {
  auto& c = *c_;
  Result<AfterReduce> r;
  r.err = c.pending();
  if (!r.ok()) return r;
  r.err = build_reduce(c, c.b, init, fn);
  if (r.ok()) r.value.c_ = c_;
  return r;
}

Result<AfterReduce> AfterReduce::Reduce(Expr init, Combiner fn) {
  auto& c = *c_;
  Result<AfterReduce> r;
  r.err = c.pending();
  if (!r.ok()) return r;
  r.err = build_reduce(c, c.b, init, fn);
  if (r.ok()) r.value.c_ = c_;
  return r;
}

Result<AfterMap> AfterReduce::Map(const std::vector<Operand>& ops, Lambda fn) {
  auto& c = *c_;
  Result<AfterMap> r;
  r.err = c.pending();
  if (!r.ok()) return r;
  Builder* b = c.b;
  Expr body;
  r.err = build_map_lambda(
      b, c_, b->tensors_, ops, fn, true, c.elem, &body, [&](const std::string& n) { return c.liveIndex(n); },
      [&](const Dim& d, const std::string& w) { return b->checkDim(d, w); });
  if (!r.ok()) return r;
  c.st.has_post = true;
  c.st.post_operands = ops;
  c.st.post_body = body;
  r.value.c_ = c_;
  return r;
}

Tail AfterMap::AsV(const std::vector<Dim>& dims) {
  auto& c = *c_;
  if (c.pending().empty()) {
    // pkg/chain.go checkAsExact: the live axes, in order (fused maps cannot reorder axes)
    std::string e;
    if (dims.size() != c.live.size()) {
      e = "piped map: as lists " + std::to_string(dims.size()) + " axes, " + std::to_string(c.live.size()) +
          " are live at this point of the chain (producer's as minus reduced axes, in order)";
    } else {
      for (size_t i = 0; i < dims.size() && e.empty(); ++i) {
        e = c.b->checkDim(dims[i], "piped map as");
        if (e.empty() && dims[i].name != c.live[i].name)
          e = "piped map: as position " + std::to_string(i) + " binds @" + dims[i].name +
              ", the incoming axis order requires @" + c.live[i].name + " (fused maps cannot reorder axes in v0)";
      }
    }
    c.deferErr(e);
  }
  c.elem = c.st.post_body.typ;
  Tail t;
  t.c_ = c_;
  return t;
}

// pkg/chain.go store
static Result<Stored> store(std::shared_ptr<Builder::Chain> cp, Builder* b, std::map<std::string, Tensor>& declared,
                            Graph& g, const Tensor& t, const std::vector<Dim>& axes,
                            const std::function<std::string(const Dim&, const std::string&)>& check_dim) {
  auto& c = *cp;
  Result<Stored> r;
  r.err = c.pending();
  if (!r.ok()) return r;
  if (t.b != b || declared.find(t.name) == declared.end()) {
    r.err = "store: tensor \"" + t.name + "\" is not declared in this builder";
    return r;
  }
  if (axes.size() != t.dims.size()) {
    r.err = "store: " + t.name + " has rank " + std::to_string(t.dims.size()) + ", got " +
            std::to_string(axes.size()) + " index axes";
    return r;
  }
  for (size_t i = 0; i < axes.size(); ++i) {
    r.err = check_dim(axes[i], "store " + t.name);
    if (!r.ok()) return r;
    if (axes[i].name != t.dims[i].name) {
      r.err = "store: index " + std::to_string(i) + " of " + t.name + " binds @" + axes[i].name + ", but dim " +
              std::to_string(i) + " of " + t.name + " is @" + t.dims[i].name;
      return r;
    }
    if (c.liveIndex(axes[i].name) < 0) {
      r.err = "store: @" + axes[i].name + " is not a live axis at this point of the chain";
      return r;
    }
  }
  c.st.out = t;
  c.st.out_axes = axes;
  c.st.elem = c.elem;
  c.stored = true;
  g.statements.push_back(c.st);
  return r;
}

// EXTENSION (pkg_ext.h): the store of a map that no reduction follows.
Result<Stored> ext::StoreMap(MidChain mid, const Tensor& t, const std::vector<Dim>& axes) {
  auto cp = mid.c_;
  Builder* b = cp->b;
  if (cp->pending().empty()) {
    if (axes.size() != cp->live.size()) {
      cp->deferErr("store of a map: the stored axes must be all " + std::to_string(cp->live.size()) + " live axes, got " +
                   std::to_string(axes.size()) + " (a map cannot drop an axis)");
    } else {
      for (size_t i = 0; i < axes.size(); ++i)
        if (axes[i].name != cp->live[i].name)
          cp->deferErr("store of a map: axis " + std::to_string(i) + " binds @" + axes[i].name + ", the live order requires @" +
                       cp->live[i].name);
    }
  }
  return store(cp, b, b->tensors_, b->g_, t, axes, [&](const Dim& d, const std::string& w) { return b->checkDim(d, w); });
}

Result<Stored> AfterReduce::StoreV(const Tensor& t, const std::vector<Dim>& axes) {
  Builder* b = c_->b;
  return store(c_, b, b->tensors_, b->g_, t, axes, [&](const Dim& d, const std::string& w) { return b->checkDim(d, w); });
}

Result<Stored> Tail::StoreV(const Tensor& t, const std::vector<Dim>& axes) {
  Builder* b = c_->b;
  return store(c_, b, b->tensors_, b->g_, t, axes, [&](const Dim& d, const std::string& w) { return b->checkDim(d, w); });
}

}  // namespace pkg
}  // namespace tcab
