// tca_syntax.cpp -- lexer, recursive-descent parser and lowering onto the builder rungs (see tca_syntax.h).
#include "tca_syntax.h"

#include "pkg_ext.h"

#include <cctype>
#include <cstdlib>
#include <cstring>
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
  enum Kind { Lit, Name, Pipe, Unary, Binary, Call, Cast, Select } kind = Lit;
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
  struct Let {
    std::string name;
    bool annotated = false;
    Param annotation;          // the written `: tensor<...>` when present
    std::vector<Stage> stages;
    int line = 0, col = 0;
  };
  std::vector<Let> lets;       // in source order; a later let may bind an earlier one as an operand
  std::string return_name;
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

  // ---- expressions: the operators of design/syntax-design.md section 2.7 with C precedence and associativity:
  //   ?:  ||  &&  |  ^  &  == !=  < <= > >=  << >>  + -  * / %  unary - + ! ~
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
      if (id == "true" || id == "false") {
        n->kind = XNode::Lit;
        n->lit_type = Elem::Bool;
        n->value = id == "true" ? 1 : 0;
        return true;
      }
      n->kind = XNode::Name;
      n->name = id;
      return true;
    }
    return fail("expected an expression, found '" + tok.text + "'");
  }
  bool unary(XNode* n) {
    for (const char* o : {"-", "+", "!", "~"}) {
      if (!is_punct(o)) continue;
      const int l = tok.line, c = tok.col;
      bump();
      XNode x;
      if (!unary(&x)) return false;
      n->kind = XNode::Unary;
      n->name = o;
      n->args = {x};
      n->line = l;
      n->col = c;
      return true;
    }
    return primary(n);
  }
  // `|` also separates the stages of a chain: inside a lambda body it is the bit operator unless the next stage
  // keyword follows it
  bool pipe_follows() const {
    Lexer probe = lx;
    const Tok t = probe.next();
    return t.kind == Tok::Ident && (t.text == "map" || t.text == "reduce");
  }
  bool binary(XNode* n, int level) {
    static const std::vector<std::vector<const char*>> ops = {{"||"}, {"&&"}, {"|"}, {"^"}, {"&"}, {"==", "!="},
                                                              {"<=", ">=", "<", ">"}, {"<<", ">>"}, {"+", "-"}, {"*", "/", "%"}};
    if (level == static_cast<int>(ops.size())) return unary(n);
    if (!binary(n, level + 1)) return false;
    for (;;) {
      const char* hit = nullptr;
      for (const char* o : ops[level])
        if (is_punct(o)) hit = o;
      if (!hit) break;
      if (std::strcmp(hit, "|") == 0 && pipe_follows()) break;
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
    if (!is_punct("?")) return true;
    const int l = tok.line, c = tok.col;
    bump();
    XNode a, b;
    if (!expr(&a) || !expect_punct(":") || !expr(&b)) return false;   // right-associative
    XNode sel;
    sel.kind = XNode::Select;
    sel.args = {*n, a, b};
    sel.line = l;
    sel.col = c;
    *n = sel;
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
        Kernel::Let let;
        let.line = tok.line;
        let.col = tok.col;
        bump();
        if (!ident(&let.name)) return false;
        for (const Kernel::Let& prev : k->lets)
          if (prev.name == let.name) return fail_at(let.line, let.col, "let '" + let.name + "' is already bound (names are immutable)");
        if (is_punct(":")) {
          bump();
          let.annotated = true;
          if (!type(&let.annotation)) return false;
        }
        if (!expect_punct("=")) return false;
        for (;;) {
          Stage st;
          if (!stage(&st)) return false;
          let.stages.push_back(st);
          if (is_punct("|")) bump(); else break;
        }
        if (!expect_punct(";")) return false;
        k->lets.push_back(let);
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
        if (n.lit_type == Elem::Bool) return b.Bool(n.value != 0);
        return b.UInt32(static_cast<uint32_t>(n.value));
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
        if (n.name == "-" && a.kind == XNode::Lit && a.lit_type == Elem::F32) return b.Float32(-static_cast<float>(a.value));
        if (n.name == "-" && a.kind == XNode::Lit && a.lit_type == Elem::I32) return b.Int32(-static_cast<int32_t>(a.value));
        if (n.name == "-" && a.kind == XNode::Name && a.name == "inf_f32" && !env.count(a.name)) return b.Float32(-__builtin_inff());
        if (n.name == "-" && a.kind == XNode::Lit && a.lit_type != Elem::F32 && a.lit_type != Elem::I32)
          return b.Neg(lower_expr(a, env, captures));
        const Expr x = lower_expr(a, env, captures);
        if (n.name == "-") return b.Neg(x);
        if (n.name == "+") return b.Pos(x);
        if (n.name == "!") return b.Not(x);
        return b.BitsNot(x);
      }
      case XNode::Binary: {
        const Expr l = lower_expr(n.args[0], env, captures);
        const Expr r = lower_expr(n.args[1], env, captures);
        if (n.name == "+") return b.Add(l, r);
        if (n.name == "-") return b.Sub(l, r);
        if (n.name == "*") return b.Mul(l, r);
        if (n.name == "/") return b.Div(l, r);
        if (n.name == "%") return b.Mod(l, r);
        if (n.name == "==") return b.Eq(l, r);
        if (n.name == "!=") return b.Ne(l, r);
        if (n.name == "<") return b.Lt(l, r);
        if (n.name == "<=") return b.Le(l, r);
        if (n.name == ">") return b.Gt(l, r);
        if (n.name == ">=") return b.Ge(l, r);
        if (n.name == "&&") return b.And(l, r);
        if (n.name == "||") return b.Or(l, r);
        if (n.name == "&") return b.BitAnd(l, r);
        if (n.name == "|") return b.BitOr(l, r);
        if (n.name == "^") return b.BitXor(l, r);
        if (n.name == "<<") return b.Shl(l, r);
        return b.Shr(l, r);
      }
      case XNode::Select: {
        const Expr c = lower_expr(n.args[0], env, captures);
        const Expr x = lower_expr(n.args[1], env, captures);
        const Expr y = lower_expr(n.args[2], env, captures);
        return b.Select(c, x, y);
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

  // One let chain: map | reduce [| reduce]* [| map], or (the added rung of pkg_ext.h) a map alone. The returned let
  // stores into the kernel's output, every other let into a Local whose type is the chain's output type
  // (design/syntax-design.md 5.1 step 5; lowering table: `let` local tensor -> b.Local + Store).
  bool lower_let(const Kernel::Let& let, bool returned) {
    if (let.stages.empty() || !let.stages[0].is_map)
      return fail(let.line, let.col, "a let chain begins with a root map");
    const Stage& root = let.stages[0];
    const bool map_only = let.stages.size() == 1;
    if (!map_only && let.stages[1].is_map)
      return fail(let.stages[1].line, let.stages[1].col, "a chain is map | reduce [| reduce]* [| map]: a second map needs a reduction before it");
    // the root `as`: explicit; else the first reduce's as-list followed by the axis it removes (section 7.4); else,
    // for a map alone, the bound dimvars in order of first appearance (section 5.1 step 2)
    std::vector<std::string> root_as_names = root.as;
    if (!root.has_as) {
      std::vector<std::string> appear;
      for (const Binding& bd : root.bindings)
        for (const std::string& d : bd.dims) {
          bool seen = false;
          for (const std::string& a : appear) seen = seen || a == d;
          if (!seen) appear.push_back(d);
        }
      if (map_only || !let.stages[1].has_as) {
        root_as_names = appear;
      } else {
        const Stage& red0 = let.stages[1];
        root_as_names = red0.as;
        int added = 0;
        for (const std::string& dv : k.dimvars) {
          bool used = false, kept = false;
          for (const std::string& d : appear) used = used || d == dv;
          for (const std::string& a : red0.as) kept = kept || a == dv;
          if (used && !kept) { root_as_names.push_back(dv); ++added; }
        }
        if (added != 1) return fail(red0.line, red0.col, "the reduce's as-list must drop exactly one axis");
      }
    }
    size_t n_reduces = 0;
    for (size_t i = 1; i < let.stages.size() && !let.stages[i].is_map; ++i) ++n_reduces;
    if (n_reduces >= root_as_names.size())
      return fail(let.line, let.col, "a fully reduced (scalar) result has no kernel class on this path");
    const std::vector<std::string> live_names(root_as_names.begin(), root_as_names.end() - static_cast<long>(n_reduces));

    // root map
    std::vector<Operand> ops;
    if (!bind_dimvars(root, &ops)) return false;
    std::vector<Dim> iters;
    for (const std::string& dv : k.dimvars) {
      bool in_chain = false;
      for (const std::string& a : root_as_names) in_chain = in_chain || a == dv;
      auto it = dimvar.find(dv);
      if (in_chain && it != dimvar.end()) iters.push_back(it->second);
    }
    if (root.params.size() != root.bindings.size())
      return fail(root.line, root.col, "root map: " + std::to_string(root.params.size()) + " lambda parameters for " +
                                           std::to_string(root.bindings.size()) + " operands (arity)");
    const std::set<std::string> caps(root.captures.begin(), root.captures.end());
    for (const std::string& c : root.captures)
      if (!scalars.count(c)) return fail(root.line, root.col, "capture '" + c + "' is not a scalar parameter of the kernel");
    Elem elem = Elem::F32;   // element type flowing out of the chain so far
    Lambda fn([&](const std::vector<Expr>& a) {
      std::map<std::string, Expr> env;
      for (size_t i = 0; i < root.params.size(); ++i) env[root.params[i].name] = a[i];
      const Expr e = lower_expr(root.body, env, caps);
      elem = e.typ;
      return e;
    });
    auto ra = b.Stmt().IterV(iters).Map(ops, fn);
    if (!ra.ok()) return fail(root.line, root.col, err.empty() ? ra.err : err.substr(err.find(": ") + 2));

    std::vector<Dim> root_as;
    if (!axes_of(root_as_names, root.line, root.col, &root_as)) return false;
    MidChain mid = ra.value.AsV(root_as);

    // reduces
    size_t si = 1;
    Result<AfterReduce> ar;
    for (; si < let.stages.size() && !let.stages[si].is_map; ++si) {
      const Stage& rs = let.stages[si];
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
    std::vector<Dim> live(root_as.begin(), root_as.end() - static_cast<long>(n_reduces));

    // a piped map, lowered before the result is declared: a Local takes the chain's final element type
    Result<AfterMap> am;
    const bool piped = si < let.stages.size();
    std::vector<Dim> pas = live;
    if (piped) {
      const Stage& pm = let.stages[si];
      if (si + 1 != let.stages.size()) return fail(pm.line, pm.col, "nothing may follow the piped map");
      std::vector<Operand> pops;
      if (!bind_dimvars(pm, &pops)) return false;
      if (pm.params.size() != pm.bindings.size() + 1)
        return fail(pm.line, pm.col, "piped map: the lambda takes the piped value plus one parameter per operand (arity)");
      const std::set<std::string> pcaps(pm.captures.begin(), pm.captures.end());
      for (const std::string& c : pm.captures)
        if (!scalars.count(c)) return fail(pm.line, pm.col, "capture '" + c + "' is not a scalar parameter of the kernel");
      Lambda pfn([&](const std::vector<Expr>& a) {
        std::map<std::string, Expr> env;
        for (size_t i = 0; i < pm.params.size(); ++i) env[pm.params[i].name] = a[i];
        const Expr e = lower_expr(pm.body, env, pcaps);
        elem = e.typ;
        return e;
      });
      am = ar.value.Map(pops, pfn);
      if (!am.ok()) return fail(pm.line, pm.col, err.empty() ? am.err : err.substr(err.find(": ") + 2));
      if (pm.has_as) {
        pas.clear();
        if (!axes_of(pm.as, pm.line, pm.col, &pas)) return false;
      }
    }

    // where the chain stores: the kernel's output for the returned let, a Local otherwise
    Tensor result;
    if (returned) {
      if (!k.ret.is_tensor) return fail(k.line, k.col, "a fully reduced (scalar) return has no kernel class on this path");
      if (k.ret.shape.size() != live_names.size())
        return fail(k.line, k.col, "the return type has rank " + std::to_string(k.ret.shape.size()) + " but the chain leaves " +
                                       std::to_string(live_names.size()) + " axes");
      result = declare_tensor(let.name, k.ret, &live_names);
    } else {
      if (let.annotated) {  // rule 24: the annotation equals the inferred type
        if (!let.annotation.is_tensor || let.annotation.shape.size() != live.size())
          return fail(let.line, let.col, "let '" + let.name + "': the annotation has rank " +
                                             std::to_string(let.annotation.shape.size()) + " but the chain leaves " +
                                             std::to_string(live.size()) + " axes");
        if (let.annotation.elem != elem)
          return fail(let.line, let.col, std::string("let '") + let.name + "': the annotation says " + ElemName(let.annotation.elem) +
                                             " but the chain yields " + ElemName(elem));
      }
      result = b.Local(let.name, elem, live);
      tensors[let.name] = result;
    }
    Result<Stored> st;
    if (piped) st = am.value.AsV(pas).StoreV(result, live);
    else if (map_only) st = ext::StoreMap(mid, result, live);
    else st = ar.value.StoreV(result, live);
    if (!st.ok()) return fail(let.line, let.col, st.err);
    return true;
  }

  bool run(ParsedKernel* out) {
    if (k.lets.empty()) return fail(k.line, k.col, "a kernel binds at least one let chain and returns one of them");
    const Kernel::Let* returned = nullptr;
    for (const Kernel::Let& l : k.lets)
      if (l.name == k.return_name) returned = &l;
    if (returned == nullptr) return fail(k.line, k.col, "'return' must name a let-bound tensor of this kernel");
    // constant extents of parameters get one dim per dimvar that subscripts them: collect the subscripts first
    std::set<std::string> bound_lets;
    for (const Kernel::Let& l : k.lets) {
      for (const Stage& st : l.stages)
        for (const Binding& bd : st.bindings) {
          const Param* decl = nullptr;
          for (const Param& p : k.params)
            if (p.is_tensor && p.name == bd.tensor) decl = &p;
          if (decl == nullptr) {
            if (bound_lets.count(bd.tensor)) continue;   // an earlier let: checked when it is bound
            return fail(bd.line, bd.col, "unknown tensor '" + bd.tensor + "'");
          }
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
      bound_lets.insert(l.name);
    }
    for (const Param& p : k.params) {
      if (p.is_tensor) declare_tensor(p.name, p, nullptr);
      else scalars[p.name] = b.ScalarParam(p.name, p.elem);
    }
    for (const Kernel::Let& l : k.lets)
      if (!lower_let(l, &l == returned)) return false;
    auto g = b.Build();
    if (!g.ok()) return fail(k.line, k.col, g.err);
    out->name = k.name;
    out->cxx_name = k.cxx_name;
    out->output = k.return_name;
    out->graph = g.value;
    return true;
  }
};

}  // namespace

namespace {

// filepath.Clean / Dir for the virtual file set ('/'-separated)
std::string clean_path(const std::string& p) {
  std::vector<std::string> parts;
  const bool abs = !p.empty() && p[0] == '/';
  size_t i = 0;
  while (i <= p.size()) {
    const size_t j = p.find('/', i);
    const std::string part = p.substr(i, j == std::string::npos ? std::string::npos : j - i);
    if (part == "..") {
      if (!parts.empty() && parts.back() != "..") parts.pop_back();
      else if (!abs) parts.push_back("..");
    } else if (!part.empty() && part != ".") {
      parts.push_back(part);
    }
    if (j == std::string::npos) break;
    i = j + 1;
  }
  std::string out = abs ? "/" : "";
  for (size_t k = 0; k < parts.size(); ++k) out += (k ? "/" : "") + parts[k];
  return out.empty() ? "." : out;
}
std::string dir_of(const std::string& p) {
  const size_t j = p.rfind('/');
  return j == std::string::npos ? "." : (j == 0 ? "/" : p.substr(0, j));
}

struct ParsedFile {
  std::vector<Kernel> kernels;
  struct Include { std::string path; int line, col; };
  std::vector<Include> includes;
};

// One file: its kernels and its include requests (unresolved).
bool parse_file(const std::string& text, const std::string& name, ParsedFile* out, std::string* err) {
  Parser p(text);
  std::string pending_cxx;
  while (p.tok.kind != Tok::End && p.err.empty()) {
    if (p.is_punct("@")) {
      p.bump();
      std::string ann;
      if (!p.ident(&ann)) break;
      if (ann == "include") {   // '@include' stringLit ';' (design/syntax-design.md: includeDecl)
        const int l = p.tok.line, c = p.tok.col;
        if (p.tok.kind != Tok::String) { p.fail("@include takes a string literal"); break; }
        out->includes.push_back({p.tok.text, l, c});
        p.bump();
        if (!p.expect_punct(";")) break;
        continue;
      }
      std::string cxx;
      if (!p.keyed(ann == "name" ? &cxx : nullptr)) break;
      if (ann == "runtime") {
        if (!p.expect_punct(";")) break;
      } else if (ann == "name") {
        pending_cxx = cxx;
      }
      continue;
    }
    Kernel k;
    if (!p.kernel(&k, pending_cxx)) break;
    pending_cxx.clear();
    out->kernels.push_back(k);
  }
  if (!p.err.empty()) {
    *err = name.empty() ? p.err : name + ":" + p.err;
    return false;
  }
  return true;
}

// internal/syntax/module.go:86-124 resolveIncludes: depth-first, an included file's kernels land after the
// including file's own, a file reached twice merges once (include guard), a file that includes one of its
// includers is a cycle; paths are relative to the including file and may not leave its directory.
struct Loader {
  const std::vector<SourceFile>& files;
  std::set<std::string> processed;
  std::string err;
  bool prefix = true;   // diagnostics carry the file's path (not for a module given as one text)

  const SourceFile* find(const std::string& path) const {
    for (const SourceFile& f : files)
      if (clean_path(f.path) == path) return &f;
    return nullptr;
  }
  bool resolve(ParsedFile* m, const std::string& path, std::set<std::string> stack) {
    for (const ParsedFile::Include& inc : m->includes) {
      auto bad = [&](const std::string& msg) {
        err = (prefix ? path + ":" : std::string()) + std::to_string(inc.line) + ":" + std::to_string(inc.col) + ": " + msg;
        return false;
      };
      if (!inc.path.empty() && inc.path[0] == '/')
        return bad("@include path \"" + inc.path + "\" must be relative to the including file");
      const std::string dir = dir_of(path);
      const std::string resolved = clean_path(dir + "/" + inc.path);
      const bool within = dir == "." ? (resolved.rfind("..", 0) != 0) : (resolved == dir || resolved.rfind(dir + "/", 0) == 0);
      if (!within) return bad("@include path \"" + inc.path + "\" escapes the including file's directory");
      const SourceFile* f = find(resolved);
      if (f == nullptr) return bad("missing include file \"" + inc.path + "\"");
      if (stack.count(resolved)) return bad("@include cycle: " + resolved + " is already being loaded");
      if (processed.count(resolved)) continue;
      ParsedFile sub;
      if (!parse_file(f->text, resolved, &sub, &err)) return false;
      processed.insert(resolved);
      std::set<std::string> inner = stack;
      inner.insert(resolved);
      if (!resolve(&sub, resolved, inner)) return false;
      m->kernels.insert(m->kernels.end(), sub.kernels.begin(), sub.kernels.end());
    }
    return true;
  }
};

Result<std::vector<ParsedKernel>> lower_all(const std::vector<Kernel>& kernels) {
  Result<std::vector<ParsedKernel>> r;
  std::set<std::string> names;
  for (const Kernel& k : kernels) {
    if (!names.insert(k.name).second) {   // module rule: kernel names are unique across the merged module
      r.err = std::to_string(k.line) + ":" + std::to_string(k.col) + ": kernel '" + k.name + "' is defined twice in the module";
      r.value.clear();
      return r;
    }
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

}  // namespace

Result<std::vector<ParsedKernel>> ParseModuleFiles(const std::vector<SourceFile>& files, const std::string& root) {
  Result<std::vector<ParsedKernel>> r;
  Loader ld{files, {}, "", files.size() > 1};
  const std::string root_path = clean_path(root);
  const SourceFile* f = ld.find(root_path);
  if (f == nullptr) {
    r.err = "cannot read source file: " + root;
    return r;
  }
  ParsedFile m;
  if (!parse_file(f->text, files.size() > 1 ? root_path : "", &m, &r.err)) return r;
  ld.processed.insert(root_path);
  if (!ld.resolve(&m, root_path, {root_path})) {
    r.err = ld.err;
    return r;
  }
  return lower_all(m.kernels);
}

Result<std::vector<ParsedKernel>> ParseModule(const std::string& text) {
  return ParseModuleFiles({SourceFile{"module.tca", text}}, "module.tca");
}

}  // namespace pkg
}  // namespace tcab
