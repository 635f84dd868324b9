// tca_syntax.cpp -- lexer, recursive-descent parser and lowering onto the builder rungs (see tca_syntax.h).
#include "tca_syntax.h"

#include <cctype>
#include <cstdlib>
#include <map>
#include <set>

namespace tcab {
namespace pkg {
namespace {

// ---- lexer -------------------------------------------------------------------------------
struct Tok {
  enum Kind { End, Ident, Int, UInt, Float, String, Punct, Pipe0 } kind = End;
  std::string text;
  double value = 0;
  int line = 1, col = 1;
};

struct Lexer {
  const std::string& s;
  size_t pos = 0;
  int line = 1, col = 1;
  std::string err;

  explicit Lexer(const std::string& src) : s(src) {}

  void adv() {
    if (s[pos] == '\n') { ++line; col = 1; } else { ++col; }
    ++pos;
  }
  void skip() {
    for (;;) {
      while (pos < s.size() && std::isspace(static_cast<unsigned char>(s[pos]))) adv();
      if (pos + 1 < s.size() && s[pos] == '/' && s[pos + 1] == '/') {
        while (pos < s.size() && s[pos] != '\n') adv();
      } else if (pos + 1 < s.size() && s[pos] == '/' && s[pos + 1] == '*') {
        adv(); adv();
        while (pos + 1 < s.size() && !(s[pos] == '*' && s[pos + 1] == '/')) adv();
        if (pos + 1 < s.size()) { adv(); adv(); }
        else { while (pos < s.size()) adv(); if (err.empty()) err = "unterminated block comment"; }
      } else {
        return;
      }
    }
  }
  Tok next() {
    skip();
    Tok t;
    t.line = line;
    t.col = col;
    if (pos >= s.size()) return t;
    const char c = s[pos];
    if (std::isalpha(static_cast<unsigned char>(c)) || c == '_') {
      size_t b = pos;
      while (pos < s.size() && (std::isalnum(static_cast<unsigned char>(s[pos])) || s[pos] == '_')) adv();
      t.kind = Tok::Ident;
      t.text = s.substr(b, pos - b);
      return t;
    }
    if (std::isdigit(static_cast<unsigned char>(c))) {
      size_t b = pos;
      bool is_float = false;
      while (pos < s.size() && std::isdigit(static_cast<unsigned char>(s[pos]))) adv();
      if (pos < s.size() && s[pos] == '.') { is_float = true; adv(); while (pos < s.size() && std::isdigit(static_cast<unsigned char>(s[pos]))) adv(); }
      if (pos < s.size() && (s[pos] == 'e' || s[pos] == 'E')) {
        is_float = true;
        adv();
        if (pos < s.size() && (s[pos] == '+' || s[pos] == '-')) adv();
        while (pos < s.size() && std::isdigit(static_cast<unsigned char>(s[pos]))) adv();
      }
      t.text = s.substr(b, pos - b);
      t.value = std::strtod(t.text.c_str(), nullptr);
      if (pos < s.size() && (s[pos] == 'f' || s[pos] == 'F')) { adv(); t.kind = Tok::Float; return t; }
      if (is_float) { err = "a float literal needs the f suffix"; t.kind = Tok::Float; return t; }
      if (pos < s.size() && (s[pos] == 'u' || s[pos] == 'U')) { adv(); t.kind = Tok::UInt; return t; }
      t.kind = Tok::Int;
      return t;
    }
    if (c == '"') {
      adv();
      size_t b = pos;
      while (pos < s.size() && s[pos] != '"') adv();
      t.kind = Tok::String;
      t.text = s.substr(b, pos - b);
      if (pos < s.size()) adv();
      else if (err.empty()) err = "unterminated string";
      return t;
    }
    if (c == '%' && pos + 1 < s.size() && std::isdigit(static_cast<unsigned char>(s[pos + 1]))) {
      adv();
      size_t b = pos;
      while (pos < s.size() && std::isdigit(static_cast<unsigned char>(s[pos]))) adv();
      t.kind = Tok::Pipe0;
      t.text = "%" + s.substr(b, pos - b);
      return t;
    }
    static const char* two[] = {"->", "==", "!=", "<=", ">=", "&&", "||", "<<", ">>"};
    for (const char* p : two)
      if (pos + 1 < s.size() && s[pos] == p[0] && s[pos + 1] == p[1]) {
        adv(); adv();
        t.kind = Tok::Punct;
        t.text = p;
        return t;
      }
    adv();
    t.kind = Tok::Punct;
    t.text = std::string(1, c);
    return t;
  }
};

// ---- AST (design/syntax-design.md section 3, the subset) ---------------------------------------
struct XNode {  // scalar expression
  enum Kind { Lit, Name, Pipe, Unary, Binary, Call, Cast } kind = Lit;
  Elem lit_type = Elem::F32;
  double value = 0;
  std::string name;  // Name / operator / builtin / cast target
  std::vector<XNode> args;
  int line = 0, col = 0;
};
struct ParamSpec { bool pipe = false; std::string name; };
struct Binding { std::string tensor; std::vector<std::string> dims; int line = 0, col = 0; };
struct Stage {
  bool is_map = true;
  std::vector<Binding> bindings;        // map
  std::vector<std::string> captures;    // map
  std::vector<ParamSpec> params;        // map lambda params / reduce on(acc, elem)
  bool has_as = false;
  std::vector<std::string> as;
  XNode init, body;
  int line = 0, col = 0;
};
struct ShapeDim { std::string name; int extent = 0; };
struct Param { std::string name; bool is_tensor = false; Elem elem = Elem::F32; std::vector<ShapeDim> shape; };
struct Kernel {
  std::string name, cxx_name;
  std::vector<Param> params;
  Param ret;
  std::vector<std::string> dimvars;
  std::string let_name, return_name;
  std::vector<Stage> stages;
  int line = 0, col = 0;
};

bool elem_from(const std::string& s, Elem* e) {
  static const std::map<std::string, Elem> m = {{"f32", Elem::F32}, {"bf16", Elem::BF16}, {"f16", Elem::F16},
                                                {"i32", Elem::I32}, {"u32", Elem::U32}, {"bool", Elem::Bool}};
  auto it = m.find(s);
  if (it == m.end()) return false;
  *e = it->second;
  return true;
}

// ---- parser -------------------------------------------------------------------------------------
struct Parser {
  Lexer lx;
  Tok tok;
  std::string err;

  explicit Parser(const std::string& src) : lx(src) { tok = lx.next(); }

  bool fail(const std::string& m) { return fail_at(tok.line, tok.col, m); }
  bool fail_at(int line, int col, const std::string& m) {
    if (err.empty()) err = std::to_string(line) + ":" + std::to_string(col) + ": " + m;
    return false;
  }
  void bump() {
    tok = lx.next();
    if (!lx.err.empty()) fail(lx.err);
  }
  bool is_punct(const char* p) const { return tok.kind == Tok::Punct && tok.text == p; }
  bool is_ident(const char* p) const { return tok.kind == Tok::Ident && tok.text == p; }
  bool expect_punct(const char* p) {
    if (!is_punct(p)) return fail(std::string("expected '") + p + "', found '" + tok.text + "'");
    bump();
    return true;
  }
  bool expect_kw(const char* p) {
    if (!is_ident(p)) return fail(std::string("expected '") + p + "', found '" + tok.text + "'");
    bump();
    return true;
  }
  bool ident(std::string* out) {
    if (tok.kind != Tok::Ident) return fail("expected an identifier, found '" + tok.text + "'");
    *out = tok.text;
    bump();
    return true;
  }
  // identifier list up to the closing token; trailing comma allowed
  bool ident_list(const char* close, std::vector<std::string>* out) {
    while (!is_punct(close)) {
      std::string id;
      if (!ident(&id)) return false;
      out->push_back(id);
      if (is_punct(",")) bump(); else break;
    }
    return expect_punct(close);
  }

  bool elem_type(Elem* e) {
    if (tok.kind != Tok::Ident || !elem_from(tok.text, e)) return fail("expected an element type, found '" + tok.text + "'");
    bump();
    return true;
  }
  bool type(Param* p) {
    if (is_ident("tensor")) {
      bump();
      p->is_tensor = true;
      if (!expect_punct("<") || !expect_kw("dtype") || !expect_punct("=") || !elem_type(&p->elem)) return false;
      if (is_punct(",")) bump();
      if (is_ident("shape")) {
        bump();
        if (!expect_punct("=") || !expect_punct("[")) return false;
        while (!is_punct("]")) {
          ShapeDim d;
          if (tok.kind == Tok::UInt) { d.extent = static_cast<int>(tok.value); d.name = "e" + tok.text; bump(); }
          else if (tok.kind == Tok::Int) return fail("a constant extent is an unsigned literal (write " + tok.text + "u)");
          else if (!ident(&d.name)) return false;
          p->shape.push_back(d);
          if (is_punct(",")) bump(); else break;
        }
        if (!expect_punct("]")) return false;
        if (is_punct(",")) bump();
      } else {
        return fail("a tensor parameter or return type needs a shape");
      }
      return expect_punct(">");
    }
    p->is_tensor = false;
    return elem_type(&p->elem);
  }

  // keyed constants of an annotation: only cxx="..." is looked at
  bool keyed(std::string* cxx) {
    if (!expect_punct("(")) return false;
    while (!is_punct(")")) {
      std::string key;
      if (!ident(&key) || !expect_punct("=")) return false;
      if (tok.kind == Tok::String && key == "cxx" && cxx) *cxx = tok.text;
      if (tok.kind == Tok::End) return fail("unterminated annotation");
      bump();
      if (is_punct(",")) bump(); else break;
    }
    return expect_punct(")");
  }

  // ---- expressions: + - * / with C precedence; everything else in the grammar is recognised and refused
  bool primary(XNode* n) {
    n->line = tok.line;
    n->col = tok.col;
    if (tok.kind == Tok::Float || tok.kind == Tok::Int || tok.kind == Tok::UInt) {
      n->kind = XNode::Lit;
      n->lit_type = tok.kind == Tok::Float ? Elem::F32 : tok.kind == Tok::Int ? Elem::I32 : Elem::U32;
      n->value = tok.value;
      bump();
      return true;
    }
    if (tok.kind == Tok::Pipe0) {
      n->kind = XNode::Pipe;
      n->name = tok.text;
      bump();
      return true;
    }
    if (is_punct("(")) {
      bump();
      if (!expr(n)) return false;
      return expect_punct(")");
    }
    if (tok.kind == Tok::Ident) {
      const std::string id = tok.text;
      Elem e;
      bump();
      if (is_punct("(")) {
        bump();
        n->kind = elem_from(id, &e) ? XNode::Cast : XNode::Call;
        n->name = id;
        while (!is_punct(")")) {
          XNode a;
          if (!expr(&a)) return false;
          n->args.push_back(a);
          if (is_punct(",")) bump(); else break;
        }
        if (!expect_punct(")")) return false;
        if (n->kind == XNode::Cast && n->args.size() != 1) return fail_at(n->line, n->col, "a cast takes one argument");
        return true;
      }
      if (id == "true" || id == "false") return fail_at(n->line, n->col, "bool expressions have no kernel class on this path");
      n->kind = XNode::Name;
      n->name = id;
      return true;
    }
    return fail("expected an expression, found '" + tok.text + "'");
  }
  bool unary(XNode* n) {
    if (is_punct("-") || is_punct("+")) {
      const bool neg = is_punct("-");
      const int l = tok.line, c = tok.col;
      bump();
      XNode x;
      if (!unary(&x)) return false;
      if (!neg) { *n = x; return true; }
      n->kind = XNode::Unary;
      n->name = "-";
      n->args = {x};
      n->line = l;
      n->col = c;
      return true;
    }
    if (is_punct("!") || is_punct("~")) return fail("operator '" + tok.text + "' has no kernel class on this path");
    return primary(n);
  }
  bool binary(XNode* n, int level) {
    static const char* ops[2][2] = {{"+", "-"}, {"*", "/"}};
    if (level == 2) return unary(n);
    if (!binary(n, level + 1)) return false;
    for (;;) {
      const char* hit = nullptr;
      for (const char* o : ops[level])
        if (is_punct(o)) hit = o;
      if (!hit) break;
      const int l = tok.line, c = tok.col;
      bump();
      XNode r;
      if (!binary(&r, level + 1)) return false;
      XNode b;
      b.kind = XNode::Binary;
      b.name = hit;
      b.args = {*n, r};
      b.line = l;
      b.col = c;
      *n = b;
    }
    return true;
  }
  bool expr(XNode* n) {
    if (!binary(n, 0)) return false;
    for (const char* o : {"?", "==", "!=", "<", "<=", ">", ">=", "&&", "||", "&", "^", "<<", ">>", "%"})
      if (is_punct(o)) return fail(std::string("operator '") + o + "' has no kernel class on this path");
    return true;
  }

  // ---- stages ---------------------------------------------------------------------------------
  bool param_spec(ParamSpec* p) {
    if (tok.kind == Tok::Pipe0) {
      if (tok.text != "%0") return fail("only %0 is a legal placeholder");
      p->pipe = true;
      p->name = "%0";
      bump();
    } else if (!ident(&p->name)) {
      return false;
    }
    if (is_punct(":")) {
      bump();
      Elem e;
      if (!elem_type(&e)) return false;
    }
    return true;
  }
  bool param_specs(std::vector<ParamSpec>* out) {
    if (!expect_punct("(")) return false;
    while (!is_punct(")")) {
      ParamSpec p;
      if (!param_spec(&p)) return false;
      out->push_back(p);
      if (is_punct(",")) bump(); else break;
    }
    return expect_punct(")");
  }
  bool as_clause(Stage* st) {
    if (!is_ident("as")) return true;
    bump();
    st->has_as = true;
    return expect_punct("(") && ident_list(")", &st->as);
  }
  bool stage(Stage* st) {
    st->line = tok.line;
    st->col = tok.col;
    if (is_ident("map")) {
      bump();
      st->is_map = true;
      if (!expect_kw("on") || !expect_punct("(")) return false;
      while (!is_punct(")")) {
        Binding b;
        b.line = tok.line;
        b.col = tok.col;
        if (!ident(&b.tensor)) return false;
        while (is_punct("[")) {
          bump();
          std::string d;
          if (!ident(&d) || !expect_punct("]")) return false;
          b.dims.push_back(d);
        }
        st->bindings.push_back(b);
        if (is_punct(",")) bump(); else break;
      }
      if (!expect_punct(")") || !as_clause(st)) return false;
      if (is_punct("[")) {
        bump();
        if (!ident_list("]", &st->captures)) return false;
      }
      if (!param_specs(&st->params)) return false;
      if (is_punct("->")) {
        bump();
        Elem e;
        if (!elem_type(&e)) return false;
      }
      return expect_punct(":") && expr(&st->body);
    }
    if (is_ident("reduce")) {
      bump();
      st->is_map = false;
      if (!expect_punct("(") || !expect_kw("init") || !expect_punct("=") || !expr(&st->init)) return false;
      if (is_punct(",")) bump();
      if (!expect_punct(")") || !expect_kw("on") || !param_specs(&st->params)) return false;
      if (st->params.size() != 2) return fail_at(st->line, st->col, "reduce: on(...) holds exactly the accumulator and the piped element");
      if (!as_clause(st)) return false;
      Elem e;
      return expect_punct("->") && elem_type(&e) && expect_punct(":") && expr(&st->body);
    }
    return fail("expected 'map' or 'reduce', found '" + tok.text + "'");
  }

  bool kernel(Kernel* k, const std::string& pending_cxx) {
    k->line = tok.line;
    k->col = tok.col;
    if (!expect_kw("kernel") || !ident(&k->name) || !expect_punct("(")) return false;
    k->cxx_name = pending_cxx.empty() ? k->name : pending_cxx;
    while (!is_punct(")")) {
      Param p;
      if (!ident(&p.name) || !expect_punct(":") || !type(&p)) return false;
      k->params.push_back(p);
      if (is_punct(",")) bump(); else break;
    }
    if (!expect_punct(")") || !expect_punct("->") || !type(&k->ret) || !expect_punct("{")) return false;
    while (!is_punct("}")) {
      if (is_ident("dimvar")) {
        bump();
        if (is_punct("(")) {
          bump();
          if (!ident_list(")", &k->dimvars)) return false;
        } else {
          for (;;) {
            std::string d;
            if (!ident(&d)) return false;
            k->dimvars.push_back(d);
            if (is_punct(",")) bump(); else break;
          }
        }
        if (!expect_punct(";")) return false;
      } else if (is_ident("let")) {
        if (!k->let_name.empty()) return fail("one let chain per kernel: several chains have no kernel class on this path");
        bump();
        if (!ident(&k->let_name)) return false;
        if (is_punct(":")) {
          bump();
          Param ignored;
          if (!type(&ignored)) return false;
        }
        if (!expect_punct("=")) return false;
        for (;;) {
          Stage st;
          if (!stage(&st)) return false;
          k->stages.push_back(st);
          if (is_punct("|")) bump(); else break;
        }
        if (!expect_punct(";")) return false;
      } else if (is_ident("return")) {
        bump();
        if (!ident(&k->return_name) || !expect_punct(";")) return false;
      } else {
        return fail("expected 'dimvar', 'let' or 'return', found '" + tok.text + "'");
      }
    }
    return expect_punct("}");
  }
};

// ---- lowering onto the rungs (internal/syntax/build/build.go:27-36 drives pkg the same way) ----------
struct Lower {
  const Kernel& k;
  Builder b;
  std::map<std::string, Dim> dims;        // shape dim name -> handle
  std::map<std::string, Tensor> tensors;
  std::map<std::string, Expr> scalars;
  std::map<std::string, Dim> dimvar;      // dimvar -> the shape dim it is bound to
  std::map<std::pair<std::string, size_t>, std::string> where;  // (tensor, position) -> dimvar subscripting it
  std::string err;

  explicit Lower(const Kernel& kk) : k(kk), b(kk.cxx_name) {}

  bool fail(int line, int col, const std::string& m) {
    if (err.empty()) err = std::to_string(line) + ":" + std::to_string(col) + ": " + m;
    return false;
  }
  // A constant extent (`4u`) becomes a dim of its own per dimvar bound to it, so that a [4u, 4u] tensor
  // iterates two distinct axes; operands that share the dimvar share the dim.
  Tensor declare_tensor(const std::string& name, const Param& p, const std::vector<std::string>* live) {
    std::vector<Dim> ds;
    for (size_t i = 0; i < p.shape.size(); ++i) {
      const ShapeDim& sd = p.shape[i];
      std::string key = sd.name;
      if (sd.extent != 0) {
        auto w = where.find({name, i});
        if (live != nullptr && i < live->size()) key = (*live)[i] + "_" + sd.name;
        else if (w != where.end()) key = w->second + "_" + sd.name;
      }
      auto it = dims.find(key);
      if (it == dims.end()) it = dims.emplace(key, b.Dim(key, sd.extent)).first;
      ds.push_back(it->second);
    }
    Tensor t = b.Tensor(name, p.elem, ds);
    tensors[name] = t;
    return t;
  }

  // names: lambda parameters first, then captured scalar parameters (design/syntax-design.md section 3: NameRef)
  Expr lower_expr(const XNode& n, const std::map<std::string, Expr>& env, const std::set<std::string>& captures) {
    auto bad = [&](const std::string& m) {
      fail(n.line, n.col, m);
      Expr e;
      e.b = &b;
      e.err = err;
      return e;
    };
    switch (n.kind) {
      case XNode::Lit:
        if (n.lit_type == Elem::F32) return b.Float32(static_cast<float>(n.value));
        if (n.lit_type == Elem::I32) return b.Int32(static_cast<int32_t>(n.value));
        return bad("u32 literals have no kernel class on this path");
      case XNode::Pipe: {
        auto it = env.find("%0");
        return it == env.end() ? bad("%0 is not a parameter of this stage") : it->second;
      }
      case XNode::Name: {
        auto it = env.find(n.name);
        if (it != env.end()) return it->second;
        if (n.name == "inf_f32") return b.Float32(__builtin_inff());
        auto sc = scalars.find(n.name);
        if (sc != scalars.end()) {
          if (!captures.count(n.name)) return bad("scalar parameter '" + n.name + "' is used but not captured: list it in [...]");
          return sc->second;
        }
        return bad("unknown name '" + n.name + "'");
      }
      case XNode::Unary: {
        const XNode& a = n.args[0];  // a negated literal stays a literal (a reduction's init must be one)
        if (a.kind == XNode::Lit && a.lit_type == Elem::F32) return b.Float32(-static_cast<float>(a.value));
        if (a.kind == XNode::Lit && a.lit_type == Elem::I32) return b.Int32(-static_cast<int32_t>(a.value));
        if (a.kind == XNode::Name && a.name == "inf_f32" && !env.count(a.name)) return b.Float32(-__builtin_inff());
        return b.Neg(lower_expr(a, env, captures));
      }
      case XNode::Binary: {
        const Expr l = lower_expr(n.args[0], env, captures);
        const Expr r = lower_expr(n.args[1], env, captures);
        if (n.name == "+") return b.Add(l, r);
        if (n.name == "-") return b.Sub(l, r);
        if (n.name == "*") return b.Mul(l, r);
        return b.Div(l, r);
      }
      case XNode::Call: {
        std::vector<Expr> args;
        for (const XNode& a : n.args) args.push_back(lower_expr(a, env, captures));
        return b.Call(n.name, args);
      }
      case XNode::Cast: {
        Elem to = Elem::F32;
        elem_from(n.name, &to);
        return b.Cast(lower_expr(n.args[0], env, captures), to);
      }
    }
    return bad("unreachable");
  }

  bool bind_dimvars(const Stage& st, std::vector<Operand>* ops) {
    for (const Binding& bd : st.bindings) {
      auto t = tensors.find(bd.tensor);
      if (t == tensors.end()) return fail(bd.line, bd.col, "unknown tensor '" + bd.tensor + "'");
      if (bd.dims.size() != t->second.dims.size())
        return fail(bd.line, bd.col, "tensor '" + bd.tensor + "' has rank " + std::to_string(t->second.dims.size()) +
                                         ", subscripted with " + std::to_string(bd.dims.size()) + " dimvars");
      Operand op;
      op.t = t->second;
      for (size_t i = 0; i < bd.dims.size(); ++i) {
        const std::string& dv = bd.dims[i];
        bool declared = false;
        for (const std::string& d : k.dimvars) declared = declared || d == dv;
        if (!declared) return fail(bd.line, bd.col, "'" + dv + "' is not a declared dimvar");
        const Dim& shape_dim = t->second.dims[i];
        auto it = dimvar.find(dv);
        if (it == dimvar.end()) {
          dimvar[dv] = shape_dim;
        } else if (it->second.name != shape_dim.name) {
          return fail(bd.line, bd.col, "dimvar '" + dv + "' is bound to shape dim " + it->second.name + " and to " +
                                           shape_dim.name + " (design/syntax-design.md 7.5: one extent per dimvar)");
        }
        op.axes.push_back(shape_dim);
      }
      ops->push_back(op);
    }
    return true;
  }
  bool axes_of(const std::vector<std::string>& names, int line, int col, std::vector<Dim>* out) {
    for (const std::string& n : names) {
      auto it = dimvar.find(n);
      if (it == dimvar.end()) return fail(line, col, "dimvar '" + n + "' in an as-list is not bound by any operand");
      out->push_back(it->second);
    }
    return true;
  }

  bool run(ParsedKernel* out) {
    if (k.let_name.empty() || k.return_name != k.let_name)
      return fail(k.line, k.col, "a kernel is one let chain followed by 'return <that let>'");
    if (k.stages.size() < 2 || !k.stages[0].is_map || k.stages[1].is_map)
      return fail(k.line, k.col, "a chain is map | reduce [| reduce]* [| map]: a store needs a reduction before it");
    const Stage& root = k.stages[0];
    const Stage& red0 = k.stages[1];
    for (const Stage& st : k.stages)
      for (const Binding& bd : st.bindings) {
        const Param* decl = nullptr;
        for (const Param& p : k.params)
          if (p.is_tensor && p.name == bd.tensor) decl = &p;
        if (decl == nullptr) return fail(bd.line, bd.col, "unknown tensor '" + bd.tensor + "'");
        if (bd.dims.size() != decl->shape.size())
          return fail(bd.line, bd.col, "tensor '" + bd.tensor + "' has rank " + std::to_string(decl->shape.size()) +
                                           ", subscripted with " + std::to_string(bd.dims.size()) + " dimvars");
        for (size_t i = 0; i < bd.dims.size(); ++i) {
          bool declared = false;
          for (const std::string& d : k.dimvars) declared = declared || d == bd.dims[i];
          if (!declared) return fail(bd.line, bd.col, "'" + bd.dims[i] + "' is not a declared dimvar");
          where[{bd.tensor, i}] = bd.dims[i];
        }
      }
    // the root `as`: explicit, or the first reduce's as-list followed by the axis it removes (section 7.4)
    std::vector<std::string> root_as_names = root.has_as ? root.as : red0.as;
    if (!root.has_as) {
      if (!red0.has_as) return fail(red0.line, red0.col, "either the root map or the reduce must carry an as-list");
      int added = 0;
      for (const std::string& dv : k.dimvars) {
        bool used = false, kept = false;
        for (const Binding& bd : root.bindings)
          for (const std::string& d : bd.dims) used = used || d == dv;
        for (const std::string& a : red0.as) kept = kept || a == dv;
        if (used && !kept) { root_as_names.push_back(dv); ++added; }
      }
      if (added != 1) return fail(red0.line, red0.col, "the reduce's as-list must drop exactly one axis");
    }
    size_t n_reduces = 0;
    for (size_t i = 1; i < k.stages.size() && !k.stages[i].is_map; ++i) ++n_reduces;
    if (n_reduces >= root_as_names.size())
      return fail(k.line, k.col, "a fully reduced (scalar) return has no kernel class on this path");
    const std::vector<std::string> live_names(root_as_names.begin(), root_as_names.end() - static_cast<long>(n_reduces));

    for (const Param& p : k.params) {
      if (p.is_tensor) declare_tensor(p.name, p, nullptr);
      else scalars[p.name] = b.ScalarParam(p.name, p.elem);
    }
    if (!k.ret.is_tensor) return fail(k.line, k.col, "a fully reduced (scalar) return has no kernel class on this path");
    if (k.ret.shape.size() != live_names.size())
      return fail(k.line, k.col, "the return type has rank " + std::to_string(k.ret.shape.size()) + " but the chain leaves " +
                                     std::to_string(live_names.size()) + " axes");
    const Tensor result = declare_tensor(k.let_name, k.ret, &live_names);

    // root map
    std::vector<Operand> ops;
    if (!bind_dimvars(root, &ops)) return false;
    std::vector<Dim> iters;
    for (const std::string& dv : k.dimvars) {
      auto it = dimvar.find(dv);
      if (it != dimvar.end()) iters.push_back(it->second);
    }
    if (root.params.size() != root.bindings.size())
      return fail(root.line, root.col, "root map: " + std::to_string(root.params.size()) + " lambda parameters for " +
                                           std::to_string(root.bindings.size()) + " operands (arity)");
    const std::set<std::string> caps(root.captures.begin(), root.captures.end());
    for (const std::string& c : root.captures)
      if (!scalars.count(c)) return fail(root.line, root.col, "capture '" + c + "' is not a scalar parameter of the kernel");
    Lambda fn([&](const std::vector<Expr>& a) {
      std::map<std::string, Expr> env;
      for (size_t i = 0; i < root.params.size(); ++i) env[root.params[i].name] = a[i];
      return lower_expr(root.body, env, caps);
    });
    auto ra = b.Stmt().IterV(iters).Map(ops, fn);
    if (!ra.ok()) return fail(root.line, root.col, err.empty() ? ra.err : err.substr(err.find(": ") + 2));

    std::vector<Dim> root_as;
    if (!axes_of(root_as_names, root.has_as ? root.line : red0.line, root.has_as ? root.col : red0.col, &root_as)) return false;
    MidChain mid = ra.value.AsV(root_as);

    // reduces
    size_t si = 1;
    Result<AfterReduce> ar;
    for (; si < k.stages.size() && !k.stages[si].is_map; ++si) {
      const Stage& rs = k.stages[si];
      const Expr init = lower_expr(rs.init, {}, {});
      Combiner comb = [&](Expr acc, Expr v) {
        std::map<std::string, Expr> env;
        env[rs.params[0].name] = acc;
        env[rs.params[1].name] = v;
        return lower_expr(rs.body, env, {});
      };
      ar = si == 1 ? mid.Reduce(init, comb) : ar.value.Reduce(init, comb);
      if (!ar.ok()) return fail(rs.line, rs.col, ar.err);
      if (!err.empty()) return false;
    }
    // live axes now: root_as minus one per reduce
    std::vector<Dim> live(root_as.begin(), root_as.end() - static_cast<long>(si - 1));

    Result<Stored> st;
    if (si < k.stages.size()) {
      const Stage& pm = k.stages[si];
      if (si + 1 != k.stages.size()) return fail(pm.line, pm.col, "nothing may follow the piped map");
      std::vector<Operand> pops;
      if (!bind_dimvars(pm, &pops)) return false;
      if (pm.params.size() != pm.bindings.size() + 1)
        return fail(pm.line, pm.col, "piped map: the lambda takes the piped value plus one parameter per operand (arity)");
      const std::set<std::string> pcaps(pm.captures.begin(), pm.captures.end());
      Lambda pfn([&](const std::vector<Expr>& a) {
        std::map<std::string, Expr> env;
        for (size_t i = 0; i < pm.params.size(); ++i) env[pm.params[i].name] = a[i];
        return lower_expr(pm.body, env, pcaps);
      });
      auto am = ar.value.Map(pops, pfn);
      if (!am.ok()) return fail(pm.line, pm.col, err.empty() ? am.err : err.substr(err.find(": ") + 2));
      std::vector<Dim> pas = live;
      if (pm.has_as) {
        pas.clear();
        if (!axes_of(pm.as, pm.line, pm.col, &pas)) return false;
      }
      st = am.value.AsV(pas).StoreV(result, live);
    } else {
      st = ar.value.StoreV(result, live);
    }
    if (!st.ok()) return fail(k.line, k.col, st.err);
    auto g = b.Build();
    if (!g.ok()) return fail(k.line, k.col, g.err);
    out->name = k.name;
    out->cxx_name = k.cxx_name;
    out->output = k.let_name;
    out->graph = g.value;
    return true;
  }
};

}  // namespace

Result<std::vector<ParsedKernel>> ParseModule(const std::string& text) {
  Result<std::vector<ParsedKernel>> r;
  Parser p(text);
  std::vector<Kernel> kernels;
  std::string pending_cxx;
  while (p.tok.kind != Tok::End && p.err.empty()) {
    if (p.is_punct("@")) {
      p.bump();
      std::string name;
      if (!p.ident(&name)) break;
      if (name == "include") {
        p.fail("@include needs a module loader; pass the included text in the same module instead");
        break;
      }
      std::string cxx;
      if (!p.keyed(name == "name" ? &cxx : nullptr)) break;
      if (name == "runtime") {
        if (!p.expect_punct(";")) break;
      } else if (name == "name") {
        pending_cxx = cxx;
      }
      continue;
    }
    Kernel k;
    if (!p.kernel(&k, pending_cxx)) break;
    pending_cxx.clear();
    kernels.push_back(k);
  }
  if (!p.err.empty()) {
    r.err = p.err;
    return r;
  }
  for (const Kernel& k : kernels) {
    Lower lw(k);
    ParsedKernel pk;
    if (!lw.run(&pk)) {
      r.err = lw.err.empty() ? "lowering failed" : lw.err;
      r.value.clear();
      return r;
    }
    r.value.push_back(pk);
  }
  return r;
}

}  // namespace pkg
}  // namespace tcab
