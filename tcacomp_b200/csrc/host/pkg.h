// pkg.h -- C++ mirror of the reference's public graph builder (pkg/builder.go, pkg/chain.go,
// pkg/expr.go) for the map | reduce | map path, plus the step the reference leaves to its compiler
// and a hand-run nvcc build: classify each built chain and launch it through the C ABI (tcab.h).
//
// The reference's host is Go; this image has no Go toolchain, so the host side above the C ABI is
// written in C++ with the same names, argument meaning and error behaviour:
//   * handles (Dim, Tensor, Expr) carry their builder; a handle from another builder is rejected
//     by the rung that consumes it (pkg/chain.go:153-176), never by a crash;
//   * handle-creating calls (Dim, Tensor, ScalarParam, Iter, As) cannot fail at the call site:
//     their violations are recorded and surfaced by the next error-returning rung or by Build
//     (pkg/builder.go:22-27);
//   * a chain is Iter -> Map -> As -> Reduce -> {Reduce | Map -> As | Store} and must pass through
//     a reduce before any store (pkg/chain.go:16-26, 433-438) -- enforced by the rung types;
//   * expression operators require identical operand types, no implicit promotion
//     (pkg/expr.go:137-176); reducers are homogeneous (pkg/chain.go:229-264).
// Go's (value, error) returns become Result<T>; `err.empty()` is Go's `err == nil`.
#pragma once

#include <functional>
#include <map>
#include <memory>
#include <string>
#include <type_traits>
#include <vector>

#include "../../../include/tcab.h"

namespace tcab {
namespace pkg {

// Element types (internal/ir/types.go:13-24), the ones this path moves.
enum class Elem { F32, BF16, F16, I32, U32, Bool };
const char* ElemName(Elem e);

template <typename T>
struct Result {
  T value{};
  std::string err;  // empty = success
  bool ok() const { return err.empty(); }
};

class Builder;
struct Dim;
struct Tensor;

struct Dim {
  Builder* b = nullptr;
  std::string name;
  int extent = 0;  // 0 = dynamic (pkg/builder.go:163)
  const std::string& Name() const { return name; }
  int Extent() const { return extent; }
};

struct Tensor {
  Builder* b = nullptr;
  std::string name;
  std::vector<Dim> dims;
  Elem elem = Elem::F32;
  bool local = false;  // declared with Builder::Local: an intermediate between two statements, not a parameter
  const std::string& Name() const { return name; }
  Elem ElemType() const { return elem; }
  int Rank() const { return static_cast<int>(dims.size()); }
};

// One structural tensor access with its axis binding: At(lhs, m, n) is lhs[@m][@n] (pkg/builder.go:115).
struct Operand {
  Tensor t;
  std::vector<Dim> axes;
};
template <typename... D>
Operand At(const Tensor& t, D... axes) {
  return Operand{t, std::vector<Dim>{axes...}};
}

// Scalar expression tree node.
struct Node {
  enum Kind { Const, Param, Scalar, Unary, Binary, Call, Cast, Select } kind = Const;
  Elem typ = Elem::F32;
  double value = 0;           // Const
  int index = 0;              // Param: lambda parameter position
  std::string name;           // Scalar: parameter name; Unary/Binary: operator spelling; Call: builtin
  std::vector<std::shared_ptr<Node>> args;
};

struct Expr {
  Builder* b = nullptr;
  std::shared_ptr<Node> node;
  Elem typ = Elem::F32;
  std::string err;  // first deferred type error, surfaced by the chain rungs (pkg/expr.go)
  bool ok() const { return err.empty(); }
};

// One stored statement: what the rungs recorded.
struct Statement {
  std::vector<Dim> iters;            // Iter(...)
  std::vector<Operand> operands;     // root map operands
  Expr map_body;                     // over Param 0..n-1
  std::vector<Dim> as;               // root As(...): the last axis is the one the first reduce removes
  struct Reduce {
    Expr init, body;                 // body over Param 0 = acc, Param 1 = value
  };
  std::vector<Reduce> reduces;
  bool has_post = false;
  std::vector<Operand> post_operands;  // piped map operands (Param 0 is the piped value)
  Expr post_body;
  Elem elem = Elem::F32;             // element type flowing out of the chain
  Tensor out;
  std::vector<Dim> out_axes;
};

struct Graph {
  std::string name;
  std::vector<Dim> dims;
  std::vector<Tensor> tensors;
  std::vector<std::pair<std::string, Elem>> scalars;
  std::vector<Statement> statements;
};

class StmtIter;
class RootMap;
class RootAs;
class MidChain;
class AfterReduce;
class AfterMap;
class Tail;
struct Stored {};
namespace ext {
Result<Stored> StoreMap(MidChain mid, const Tensor& t, const std::vector<Dim>& axes);  // the one added rung: pkg_ext.h
}

// A map lambda: a callable of 1-4 Expr parameters (its arity is checked against the operand count,
// pkg/chain.go coerceMapFn) or of one std::vector<Expr> (variadic, any arity).
struct Lambda {
  int arity = -1;  // -1 = variadic
  std::function<Expr(const std::vector<Expr>&)> call;
  Lambda() = default;
  template <class F, std::enable_if_t<std::is_invocable_r<Expr, F, const std::vector<Expr>&>::value, int> = 0>
  Lambda(F f) : arity(-1), call(f) {}
  template <class F, std::enable_if_t<std::is_invocable_r<Expr, F, Expr>::value, int> = 0>
  Lambda(F f) : arity(1), call([f](const std::vector<Expr>& a) { return f(a[0]); }) {}
  template <class F, std::enable_if_t<std::is_invocable_r<Expr, F, Expr, Expr>::value, int> = 0>
  Lambda(F f) : arity(2), call([f](const std::vector<Expr>& a) { return f(a[0], a[1]); }) {}
  template <class F, std::enable_if_t<std::is_invocable_r<Expr, F, Expr, Expr, Expr>::value, int> = 0>
  Lambda(F f) : arity(3), call([f](const std::vector<Expr>& a) { return f(a[0], a[1], a[2]); }) {}
  template <class F, std::enable_if_t<std::is_invocable_r<Expr, F, Expr, Expr, Expr, Expr>::value, int> = 0>
  Lambda(F f) : arity(4), call([f](const std::vector<Expr>& a) { return f(a[0], a[1], a[2], a[3]); }) {}
};
using Combiner = std::function<Expr(Expr acc, Expr v)>;

class Builder {
 public:
  explicit Builder(std::string name);
  Builder(const Builder&) = delete;
  Builder& operator=(const Builder&) = delete;

  // Declarations (pkg/builder.go:163-295). Violations are deferred (see the header comment).
  // (Dim and Tensor are also the handle types, hence the qualified spellings inside this class.)
  pkg::Dim Dim(const std::string& name, int extent);
  pkg::Tensor Tensor(const std::string& name, Elem elem, const std::vector<pkg::Dim>& dims);
  template <typename... D>
  pkg::Tensor Tensor(const std::string& name, Elem elem, pkg::Dim d0, D... rest) {
    return Tensor(name, elem, std::vector<pkg::Dim>{d0, rest...});
  }
  // pkg/builder.go:224 Local: a tensor handle that one statement stores into and a later one reads as an
  // operand (the lowering of a `let` that is not the returned one). A rank-1 local may have a dynamic extent; a
  // local of rank >= 2 must be fully static ("a multiplicative GMEM size is not constructed").
  pkg::Tensor Local(const std::string& name, Elem elem, const std::vector<pkg::Dim>& dims);
  Expr ScalarParam(const std::string& name, Elem elem);
  StmtIter Stmt();
  Result<Graph> Build();  // pkg/builder.go:340-370

  // Typed scalar expression DSL (pkg/expr.go:179-341), operand classes as pkg/expr.go:137-176:
  // arithmetic operators take one arithmetic type, % and the bit operators one integer type, comparisons any
  // one type and yield bool, And / Or / Not take bool; nothing is promoted implicitly.
  Expr Add(Expr x, Expr y);
  Expr Sub(Expr x, Expr y);
  Expr Mul(Expr x, Expr y);
  Expr Div(Expr x, Expr y);
  Expr Mod(Expr x, Expr y);
  Expr Eq(Expr x, Expr y);
  Expr Ne(Expr x, Expr y);
  Expr Lt(Expr x, Expr y);
  Expr Le(Expr x, Expr y);
  Expr Gt(Expr x, Expr y);
  Expr Ge(Expr x, Expr y);
  Expr And(Expr x, Expr y);
  Expr Or(Expr x, Expr y);
  Expr BitAnd(Expr x, Expr y);
  Expr BitOr(Expr x, Expr y);
  Expr BitXor(Expr x, Expr y);
  Expr Shl(Expr x, Expr y);
  Expr Shr(Expr x, Expr y);
  Expr Neg(Expr x);
  Expr Pos(Expr x);
  Expr Not(Expr x);
  Expr BitsNot(Expr x);
  Expr Float32(float v);
  Expr Int32(int32_t v);
  Expr UInt32(uint32_t v);
  Expr Bool(bool v);
  Expr Select(Expr cond, Expr a, Expr b);  // pkg/expr.go:271: the lazy conditional cond ? a : b
  Expr Cast(Expr x, Elem to);
  Expr Call(const std::string& builtin, const std::vector<Expr>& args);  // internal/ir/builtins.go:25-39

  struct Chain;  // the statement chain under construction (implementation detail of the rungs)

 private:
  friend class StmtIter;
  friend class RootMap;
  friend class RootAs;
  friend class MidChain;
  friend class AfterReduce;
  friend class AfterMap;
  friend class Tail;
  friend Result<Stored> ext::StoreMap(MidChain mid, const pkg::Tensor& t, const std::vector<pkg::Dim>& axes);
  void noteDeclErr(const std::string& e);
  std::string checkDim(const pkg::Dim& d, const std::string& what) const;
  Expr bad(const std::string& e);
  Expr binop(const char* op, Expr x, Expr y, const char* cls = "arithmetic");
  Expr unop(const char* op, Expr x, const char* cls);

  Graph g_;
  std::map<std::string, pkg::Dim> dims_;
  std::map<std::string, pkg::Tensor> tensors_;
  std::map<std::string, Elem> scalars_;
  std::shared_ptr<Chain> chain_;
  bool final_ = false;
  std::string decl_err_;
};

// The typestate rungs (pkg/chain.go:354-559).
class StmtIter {
 public:
  template <typename... D>
  RootMap Iter(D... dims);
  RootMap IterV(const std::vector<Dim>& dims);

 private:
  friend class Builder;
  std::shared_ptr<Builder::Chain> c_;
};
class RootMap {
 public:
  Result<RootAs> Map(const std::vector<Operand>& ops, Lambda fn);

 private:
  friend class StmtIter;
  std::shared_ptr<Builder::Chain> c_;
};
class RootAs {
 public:
  template <typename... D>
  MidChain As(D... dims);
  MidChain AsV(const std::vector<Dim>& dims);

 private:
  friend class RootMap;
  std::shared_ptr<Builder::Chain> c_;
};
class AfterReduce {
 public:
  Result<AfterReduce> Reduce(Expr init, Combiner fn);
  Result<AfterMap> Map(const std::vector<Operand>& ops, Lambda fn);
  template <typename... D>
  Result<Stored> Store(const Tensor& t, D... axes);
  Result<Stored> StoreV(const Tensor& t, const std::vector<Dim>& axes);

 private:
  friend class MidChain;
  std::shared_ptr<Builder::Chain> c_;
};
class MidChain {
 public:
  Result<AfterReduce> Reduce(Expr init, Combiner fn);

 private:
  friend class RootAs;
  friend Result<Stored> ext::StoreMap(MidChain mid, const Tensor& t, const std::vector<Dim>& axes);
  std::shared_ptr<Builder::Chain> c_;
};
class Tail {
 public:
  template <typename... D>
  Result<Stored> Store(const Tensor& t, D... axes);
  Result<Stored> StoreV(const Tensor& t, const std::vector<Dim>& axes);

 private:
  friend class AfterMap;
  std::shared_ptr<Builder::Chain> c_;
};
class AfterMap {
 public:
  template <typename... D>
  Tail As(D... dims);
  Tail AsV(const std::vector<Dim>& dims);

 private:
  friend class AfterReduce;
  std::shared_ptr<Builder::Chain> c_;
};

template <typename... D>
RootMap StmtIter::Iter(D... dims) { return IterV(std::vector<Dim>{dims...}); }
template <typename... D>
MidChain RootAs::As(D... dims) { return AsV(std::vector<Dim>{dims...}); }
template <typename... D>
Result<Stored> AfterReduce::Store(const Tensor& t, D... axes) { return StoreV(t, std::vector<Dim>{axes...}); }
template <typename... D>
Result<Stored> Tail::Store(const Tensor& t, D... axes) { return StoreV(t, std::vector<Dim>{axes...}); }
template <typename... D>
Tail AfterMap::As(D... dims) { return AsV(std::vector<Dim>{dims...}); }

// ---------------------------------------------------------------------------
// Classification and launch: what replaces compile + emit + nvcc + <Name>Launch.
// ---------------------------------------------------------------------------

// Prints a lambda body as the C expression text the C ABI takes: lambda parameters become p0..,
// scalar parameters c0.. (slots assigned in order of first appearance and appended to `captures`),
// literals keep their value. `first_param` shifts parameter numbering (a piped map's parameter 0 is
// the piped value).
std::string PrintLambda(const Expr& body, std::vector<std::string>* captures);

struct Plan {
  enum Kind { ChainReduce, ChainContract, GemmBiasAct, Map, SoftmaxRows, LayernormRows } kind = ChainReduce;
  // ChainReduce
  std::string map_expr, combine_expr, post_expr;
  float init = 0.0f;
  std::vector<std::string> capture_names;  // scalar parameter of capture slot i
  std::vector<std::string> inputs;         // tensor names, in operand order
  uint32_t reduce_axis = 0;                // position of the reduced dim in the operands
  bool rhs_is_nk = false;                  // ChainContract: the second operand is [n,k] rather than [k,n]
  // ChainReduce / Map: how operand i is indexed -- 0 by every axis, 1 one value per row (it lacks the innermost
  // axis), 2 one row shared by all rows (it has the innermost axis only), 3 one value per output cell (it lacks
  // the reduced axis, which is not the innermost)
  std::vector<int> indexing;
  // GemmBiasAct
  std::string a, b, bias;                  // bias empty = none
  int act = TCAB_ACT_NONE;
  // SoftmaxRows: inputs = {x}; LayernormRows: inputs = {x, gamma, beta}, eps_scalar names the scalar parameter
  std::string eps_scalar;
  std::string out;
  std::vector<std::string> fused_locals;   // locals of the statements this plan replaces: they need no memory
};

// Matches a statement to an operator class of the kernel library; err explains a chain no class covers.
Result<Plan> Classify(const Statement& st);

// The launches a graph lowers to, in order: every statement classified, after the statement groups that spell
// a whole row chain -- max into a local, sum of exp(x - max) into a local, the normalising map (row softmax);
// mean and variance into locals, the scale-and-shift map (layer-norm) -- have been replaced by the one-launch
// operators tcab_softmax_rows / tcab_layernorm_rows. err names the first statement no class covers.
Result<std::vector<Plan>> PlanGraph(const Graph& g);

// Device bindings for a launch: the C spelling of the tca::Tensor arguments of the generated
// launcher (internal/cg/cxx/launch.go:23-156), by tensor name; scalars by parameter name.
struct Bindings {
  std::map<std::string, tcab_tensor> tensors;
  std::map<std::string, float> scalars;
};

// Launches every statement of the graph in order on `stream`. Like the generated launcher it derives
// each dim from its first tensor occurrence and requires every other occurrence to agree, by name.
// Returns a tcab_status; message() of the failure through LastError().
int Launch(const Graph& g, const Bindings& bind, void* stream);
const std::string& LastError();

}  // namespace pkg
}  // namespace tcab
