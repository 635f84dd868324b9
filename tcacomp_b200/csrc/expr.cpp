// expr.cpp -- typed recursive-descent parser for the lambda expressions (see expr.h).
#include "expr.h"

#include <cctype>
#include <cerrno>
#include <cstdlib>
#include <cstring>

namespace tcab {

const char* elem_name(ElemT t) {
  switch (t) {
    case kF32: return "f32";
    case kBF16: return "bf16";
    case kI32: return "i32";
    case kU32: return "u32";
    default: return "bool";
  }
}

const char* elem_cxx(ElemT t) {
  switch (t) {
    case kF32: return "float";
    case kBF16: return "__nv_bfloat16";
    case kI32: return "int32_t";
    case kU32: return "uint32_t";
    default: return "bool";
  }
}

namespace {

struct Builtin {
  const char* name;
  int arity;
  ElemT type;  // argument and result type (internal/ir/builtins.go:25-39)
};
// internal/ir/builtins.go:25-39 / internal/cg/cxx/naming.go:188-198: the f32 builtins are emitted verbatim (CUDA's
// math library); umin / umax are the reference's u32 pair (runtime/tca/mapping.h:38-39), CUDA's functions of that name.
const Builtin kBuiltins[] = {{"expf", 1, kF32},  {"logf", 1, kF32},  {"sqrtf", 1, kF32}, {"rsqrtf", 1, kF32},
                             {"fabsf", 1, kF32}, {"tanhf", 1, kF32}, {"sinf", 1, kF32},  {"cosf", 1, kF32},
                             {"fminf", 2, kF32}, {"fmaxf", 2, kF32}, {"fmaf", 3, kF32},  {"umin", 2, kU32},
                             {"umax", 2, kU32}};

struct TypeName {
  const char* name;
  ElemT type;
};
const TypeName kTypeNames[] = {{"f32", kF32},      {"float", kF32},  {"bf16", kBF16},    {"__nv_bfloat16", kBF16},
                               {"i32", kI32},      {"int32_t", kI32}, {"int", kI32},     {"u32", kU32},
                               {"uint32_t", kU32}, {"unsigned", kU32}};

bool is_int(ElemT t) { return t == kI32 || t == kU32; }
bool is_arith(ElemT t) { return t == kF32 || is_int(t); }  // bf16 is a storage type: convert first

struct Val {
  std::string text;
  ElemT type = kF32;
};

struct Parser {
  const char* s;
  size_t pos = 0;
  int max_operands;
  const ElemT* operand_types;
  size_t n_user;
  CanonExpr* out;
  std::string err;
  int depth = 0;

  void skip() {
    while (s[pos] && std::isspace(static_cast<unsigned char>(s[pos]))) ++pos;
  }
  bool fail(const std::string& m) {
    if (err.empty()) err = m + " at offset " + std::to_string(pos);
    return false;
  }
  bool at(const char* tok) {
    skip();
    return std::strncmp(s + pos, tok, std::strlen(tok)) == 0;
  }
  bool eat(const char* tok) {
    if (!at(tok)) return false;
    pos += std::strlen(tok);
    return true;
  }
  int lift(float v) {
    // Equal bit patterns share a slot; only lifted slots are searched, so a user capture is never aliased.
    for (size_t i = n_user; i < out->captures.size(); ++i)
      if (std::memcmp(&out->captures[i], &v, sizeof(float)) == 0) return static_cast<int>(i);
    out->captures.push_back(v);
    return static_cast<int>(out->captures.size() - 1);
  }
  struct Nest {
    Parser* p;
    bool ok;
    explicit Nest(Parser* q) : p(q), ok(++q->depth <= 64) {
      if (!ok) p->fail("expression nests too deeply");
    }
    ~Nest() { --p->depth; }
  };

  bool binary_type(const char* op, const Val& a, const Val& b, const char* cls, ElemT* result) {
    if (a.type != b.type)
      return fail(std::string("operator ") + op + ": operand types differ (" + elem_name(a.type) + " vs " + elem_name(b.type) +
                  "); implicit promotions are not supported");
    const ElemT t = a.type;
    if (!std::strcmp(cls, "arith")) {
      if (!is_arith(t)) return fail(std::string("operator ") + op + ": operands must have an arithmetic type (convert bf16 to f32 first), got " + elem_name(t));
      *result = t;
    } else if (!std::strcmp(cls, "int")) {
      if (!is_int(t)) return fail(std::string("operator ") + op + ": operands must have the same integer type, got " + elem_name(t));
      *result = t;
    } else if (!std::strcmp(cls, "bool")) {
      if (t != kBool) return fail(std::string("operator ") + op + ": operands must be bool, got " + elem_name(t));
      *result = kBool;
    } else {  // comparison
      if (t == kBF16) return fail(std::string("operator ") + op + ": bf16 is a storage type, convert to f32 first");
      *result = kBool;
    }
    return true;
  }

  // One left-associative level: operators `ops` (longest first), operand class `cls`, next level `next`.
  template <class Next>
  bool level(Val* r, const char* const* ops, int n_ops, const char* cls, Next next, const char* const* not_followed_by = nullptr) {
    if (!next(r)) return false;
    for (;;) {
      skip();
      const char* hit = nullptr;
      for (int i = 0; i < n_ops && !hit; ++i) {
        const size_t len = std::strlen(ops[i]);
        if (std::strncmp(s + pos, ops[i], len) != 0) continue;
        bool blocked = false;  // "&" must not eat the first half of "&&", "<" not that of "<<" or "<="
        if (not_followed_by)
          for (const char* const* nf = not_followed_by; *nf && !blocked; ++nf) blocked = s[pos + len] == **nf;
        if (!blocked) hit = ops[i];
      }
      if (!hit) return true;
      pos += std::strlen(hit);
      Val b;
      if (!next(&b)) return false;
      ElemT t;
      if (!binary_type(hit, *r, b, cls, &t)) return false;
      r->text = "(" + r->text + " " + hit + " " + b.text + ")";
      r->type = t;
    }
  }

  bool primary(Val* r) {
    Nest n(this);
    if (!n.ok) return false;
    skip();
    const char c = s[pos];
    if (c == '(') {
      ++pos;
      if (!ternary(r)) return false;
      skip();
      if (s[pos] != ')') return fail("expected ')'");
      ++pos;
      return true;
    }
    if (std::isdigit(static_cast<unsigned char>(c)) || (c == '.' && std::isdigit(static_cast<unsigned char>(s[pos + 1])))) return number(r);
    if (std::isalpha(static_cast<unsigned char>(c)) || c == '_') return identifier(r);
    return fail("unexpected character");
  }

  bool number(Val* r) {
    size_t e = pos;
    bool floating = false;
    while (std::isdigit(static_cast<unsigned char>(s[e]))) ++e;
    if (s[e] == '.') {
      floating = true;
      ++e;
      while (std::isdigit(static_cast<unsigned char>(s[e]))) ++e;
    }
    if (s[e] == 'e' || s[e] == 'E') {
      size_t x = e + 1;
      if (s[x] == '+' || s[x] == '-') ++x;
      if (std::isdigit(static_cast<unsigned char>(s[x]))) {
        floating = true;
        e = x;
        while (std::isdigit(static_cast<unsigned char>(s[e]))) ++e;
      }
    }
    if (floating || s[e] == 'f' || s[e] == 'F') {  // f32 literal: lifted into a capture slot
      char* end = nullptr;
      const float v = std::strtof(s + pos, &end);
      if (end == s + pos) return fail("bad number");
      pos = static_cast<size_t>(end - s);
      if (s[pos] == 'f' || s[pos] == 'F') ++pos;
      r->text = "c" + std::to_string(lift(v));
      r->type = kF32;
      return true;
    }
    errno = 0;
    char* end = nullptr;
    const unsigned long long v = std::strtoull(s + pos, &end, 10);
    if (end == s + pos || errno == ERANGE) return fail("bad integer literal");
    pos = static_cast<size_t>(end - s);
    if (s[pos] == 'u' || s[pos] == 'U') {  // u32 literal (pkg/expr.go UInt32)
      ++pos;
      if (v > 0xffffffffull) return fail("u32 literal out of range");
      r->text = std::to_string(v) + "u";
      r->type = kU32;
    } else {  // decimal integers are i32 (pkg/expr.go Int32); the sign is a separate operator
      if (v > 0x7fffffffull) return fail("i32 literal out of range");
      r->text = std::to_string(v);
      r->type = kI32;
    }
    if (std::isalnum(static_cast<unsigned char>(s[pos])) || s[pos] == '_' || s[pos] == '.') return fail("bad number");
    return true;
  }

  bool call_args(const std::string& id, int arity, ElemT want, std::string* args) {
    skip();
    if (s[pos] != '(') return fail("expected '(' after " + id);
    ++pos;
    for (int a = 0; a < arity; ++a) {
      Val e;
      if (!ternary(&e)) return false;
      if (e.type != want) return fail("call " + id + ": argument " + std::to_string(a) + " must be " + elem_name(want) + ", got " + elem_name(e.type));
      skip();
      if (a + 1 < arity) {
        if (s[pos] != ',') return fail(id + " takes " + std::to_string(arity) + " argument(s)");
        ++pos;
        *args += e.text + ", ";
      } else {
        *args += e.text;
      }
    }
    if (s[pos] != ')') return fail("expected ')' closing " + id);
    ++pos;
    return true;
  }

  bool cast_to(ElemT to, Val* r) {  // the '(' operand ')' part of a conversion
    skip();
    if (s[pos] != '(') return fail("expected '(' after the conversion's type");
    ++pos;
    Val e;
    if (!ternary(&e)) return false;
    skip();
    if (s[pos] != ')') return fail("expected ')' closing the conversion");
    ++pos;
    if (e.type == kBool) return fail("cast: bool cannot be converted (arithmetic-to-arithmetic only)");
    if (e.type == to) return fail(std::string("cast: redundant cast to ") + elem_name(to));
    r->text = std::string("static_cast<") + elem_cxx(to) + ">(" + e.text + ")";
    r->type = to;
    return true;
  }

  bool identifier(Val* r) {
    const size_t b = pos;
    while (std::isalnum(static_cast<unsigned char>(s[pos])) || s[pos] == '_') ++pos;
    const std::string id(s + b, pos - b);
    if ((id[0] == 'p' || id[0] == 'c') && id.size() > 1 && id.size() < 4 && std::isdigit(static_cast<unsigned char>(id[1])) &&
        (id.size() == 2 || std::isdigit(static_cast<unsigned char>(id[2])))) {
      const int idx = std::atoi(id.c_str() + 1);
      if (id[0] == 'p') {
        if (idx >= max_operands) return fail("operand " + id + " out of range");
        if (idx + 1 > out->n_operands) out->n_operands = idx + 1;
        r->type = operand_types ? operand_types[idx] : kF32;
      } else {
        if (static_cast<size_t>(idx) >= n_user) return fail("capture " + id + " out of range");
        r->type = kF32;
      }
      r->text = id;
      return true;
    }
    if (id == "true" || id == "false") {
      r->text = id;
      r->type = kBool;
      return true;
    }
    if (id == "static_cast") {
      skip();
      if (s[pos] != '<') return fail("expected '<' after static_cast");
      ++pos;
      skip();
      const size_t tb = pos;
      while (std::isalnum(static_cast<unsigned char>(s[pos])) || s[pos] == '_') ++pos;
      const std::string tn(s + tb, pos - tb);
      skip();
      if (s[pos] != '>') return fail("expected '>' after the conversion's type");
      ++pos;
      for (const TypeName& t : kTypeNames)
        if (tn == t.name) return cast_to(t.type, r);
      return fail("cast: unknown target type '" + tn + "'");
    }
    for (const TypeName& t : kTypeNames)
      if (id == t.name) return cast_to(t.type, r);
    for (const Builtin& bi : kBuiltins) {
      if (id != bi.name) continue;
      std::string args;
      if (!call_args(id, bi.arity, bi.type, &args)) return false;
      r->text = id + "(" + args + ")";
      r->type = bi.type;
      return true;
    }
    return fail("unknown identifier '" + id + "'");
  }

  bool unary(Val* r) {
    Nest n(this);
    if (!n.ok) return false;
    skip();
    const char c = s[pos];
    if (c == '-' || c == '+' || c == '!' || c == '~') {
      ++pos;
      Val a;
      if (!unary(&a)) return false;
      if ((c == '-' || c == '+') && !is_arith(a.type)) return fail(std::string("unary ") + c + ": operand must have an arithmetic type, got " + elem_name(a.type));
      if (c == '!' && a.type != kBool) return fail(std::string("unary !: operand must be bool, got ") + elem_name(a.type));
      if (c == '~' && !is_int(a.type)) return fail(std::string("unary ~: operand must have an integer type, got ") + elem_name(a.type));
      r->text = c == '+' ? a.text : std::string("(") + c + a.text + ")";
      r->type = a.type;
      return true;
    }
    return primary(r);
  }

  bool mul(Val* r) {
    // % is in the integer group (pkg/expr.go:191); * and / take any arithmetic type
    if (!unary(r)) return false;
    for (;;) {
      skip();
      const char c = s[pos];
      if (c != '*' && c != '/' && c != '%') return true;
      ++pos;
      Val b;
      if (!unary(&b)) return false;
      ElemT t;
      const char op[2] = {c, 0};
      if (!binary_type(op, *r, b, c == '%' ? "int" : "arith", &t)) return false;
      r->text = "(" + r->text + " " + c + " " + b.text + ")";
      r->type = t;
    }
  }
  bool add(Val* r) {
    static const char* const ops[] = {"+", "-"};
    return level(r, ops, 2, "arith", [this](Val* v) { return mul(v); });
  }
  bool shift(Val* r) {
    static const char* const ops[] = {"<<", ">>"};
    return level(r, ops, 2, "int", [this](Val* v) { return add(v); });
  }
  bool rel(Val* r) {
    static const char* const ops[] = {"<=", ">=", "<", ">"};
    static const char* const nf[] = {"<", ">", nullptr};  // "<" is not the first half of "<<"
    return level(r, ops, 4, "cmp", [this](Val* v) { return shift(v); }, nf);
  }
  bool eq(Val* r) {
    static const char* const ops[] = {"==", "!="};
    return level(r, ops, 2, "cmp", [this](Val* v) { return rel(v); });
  }
  bool band(Val* r) {
    static const char* const ops[] = {"&"};
    static const char* const nf[] = {"&", nullptr};
    return level(r, ops, 1, "int", [this](Val* v) { return eq(v); }, nf);
  }
  bool bxor(Val* r) {
    static const char* const ops[] = {"^"};
    return level(r, ops, 1, "int", [this](Val* v) { return band(v); });
  }
  bool bor(Val* r) {
    static const char* const ops[] = {"|"};
    static const char* const nf[] = {"|", nullptr};
    return level(r, ops, 1, "int", [this](Val* v) { return bxor(v); }, nf);
  }
  bool land(Val* r) {
    static const char* const ops[] = {"&&"};
    return level(r, ops, 1, "bool", [this](Val* v) { return bor(v); });
  }
  bool lor(Val* r) {
    static const char* const ops[] = {"||"};
    return level(r, ops, 1, "bool", [this](Val* v) { return land(v); });
  }
  bool ternary(Val* r) {
    Nest n(this);
    if (!n.ok) return false;
    if (!lor(r)) return false;
    skip();
    if (s[pos] != '?') return true;
    ++pos;
    if (r->type != kBool) return fail(std::string("select: condition must be bool, got ") + elem_name(r->type));
    Val a, b;
    if (!ternary(&a)) return false;
    skip();
    if (s[pos] != ':') return fail("expected ':' in a conditional");
    ++pos;
    if (!ternary(&b)) return false;
    if (a.type != b.type)
      return fail(std::string("select: branches must have identical types, got ") + elem_name(a.type) + " vs " + elem_name(b.type));
    r->text = "(" + r->text + " ? " + a.text + " : " + b.text + ")";  // internal/cg/cxx/expr.go:38-56
    r->type = a.type;
    return true;
  }
};

}  // namespace

bool canonicalize(const char* src, int max_operands, const ElemT* operand_types, const std::vector<float>& user_captures,
                  CanonExpr* out, std::string* err) {
  if (src == nullptr) {
    if (err) *err = "null expression";
    return false;
  }
  if (std::strlen(src) > 4096) {
    if (err) *err = "expression longer than 4096 characters";
    return false;
  }
  out->text.clear();
  out->captures = user_captures;
  out->n_operands = 0;
  Parser p{src, 0, max_operands, operand_types, user_captures.size(), out, {}, 0};
  Val v;
  bool ok = p.ternary(&v);
  if (ok) {
    p.skip();
    if (src[p.pos] != '\0') ok = p.fail("trailing characters");
  }
  if (!ok) {
    if (err) *err = p.err;
    return false;
  }
  out->type = v.type;
  const std::string& r = v.text;
  // Renumber the captures in order of first appearance and drop the unused ones, so that the
  // canonical text does not depend on how many captures the caller declared.
  std::vector<int> remap(out->captures.size(), -1);
  std::vector<float> compact;
  std::string text;
  for (size_t i = 0; i < r.size();) {
    const bool ident_start = r[i] == 'c' && (i == 0 || !(std::isalnum(static_cast<unsigned char>(r[i - 1])) || r[i - 1] == '_')) &&
                             i + 1 < r.size() && std::isdigit(static_cast<unsigned char>(r[i + 1]));
    if (!ident_start) {
      text += r[i++];
      continue;
    }
    size_t j = i + 1;
    while (j < r.size() && std::isdigit(static_cast<unsigned char>(r[j]))) ++j;
    const int old = std::atoi(r.c_str() + i + 1);
    if (remap[old] < 0) {
      remap[old] = static_cast<int>(compact.size());
      compact.push_back(out->captures[old]);
    }
    text += "c" + std::to_string(remap[old]);
    i = j;
  }
  out->text = text;
  out->captures = compact;
  return true;
}

}  // namespace tcab
