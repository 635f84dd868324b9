// expr.cpp -- recursive-descent parser for the lambda expressions (see expr.h).
#include "expr.h"

#include <cctype>
#include <cstdlib>
#include <cstring>

namespace tcab {
namespace {

struct Builtin {
  const char* name;
  int arity;
};
// internal/ir/builtins.go:25-39 / internal/cg/cxx/naming.go:188-198: the fp32 builtins, emitted verbatim.
const Builtin kBuiltins[] = {{"expf", 1},  {"logf", 1}, {"sqrtf", 1}, {"rsqrtf", 1}, {"fabsf", 1},
                             {"tanhf", 1}, {"sinf", 1}, {"cosf", 1},  {"fminf", 2},  {"fmaxf", 2},
                             {"fmaf", 3}};

struct Parser {
  const char* s;
  size_t pos = 0;
  int max_operands;
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
  int lift(float v) {
    // Equal bit patterns share a slot; only lifted slots are searched, so a user capture is never aliased.
    for (size_t i = n_user; i < out->captures.size(); ++i)
      if (std::memcmp(&out->captures[i], &v, sizeof(float)) == 0) return static_cast<int>(i);
    out->captures.push_back(v);
    return static_cast<int>(out->captures.size() - 1);
  }

  bool primary(std::string* r) {
    skip();
    if (++depth > 64) return fail("expression nests too deeply");
    bool ok = primary_inner(r);
    --depth;
    return ok;
  }
  bool primary_inner(std::string* r) {
    const char c = s[pos];
    if (c == '(') {
      ++pos;
      if (!additive(r)) return false;
      skip();
      if (s[pos] != ')') return fail("expected ')'");
      ++pos;
      return true;
    }
    if (c == '-' || c == '+') {
      ++pos;
      std::string a;
      if (!primary(&a)) return false;
      *r = c == '-' ? "(-" + a + ")" : a;
      return true;
    }
    if (std::isdigit(static_cast<unsigned char>(c)) || c == '.') {
      char* end = nullptr;
      const float v = std::strtof(s + pos, &end);
      if (end == s + pos) return fail("bad number");
      pos = static_cast<size_t>(end - s);
      if (s[pos] == 'f' || s[pos] == 'F') ++pos;
      *r = "c" + std::to_string(lift(v));
      return true;
    }
    if (std::isalpha(static_cast<unsigned char>(c)) || c == '_') {
      size_t b = pos;
      while (std::isalnum(static_cast<unsigned char>(s[pos])) || s[pos] == '_') ++pos;
      const std::string id(s + b, pos - b);
      if ((id[0] == 'p' || id[0] == 'c') && id.size() > 1 && id.size() < 4 &&
          std::isdigit(static_cast<unsigned char>(id[1])) &&
          (id.size() == 2 || std::isdigit(static_cast<unsigned char>(id[2])))) {
        const int idx = std::atoi(id.c_str() + 1);
        if (id[0] == 'p') {
          if (idx >= max_operands) return fail("operand " + id + " out of range");
          if (idx + 1 > out->n_operands) out->n_operands = idx + 1;
        } else if (static_cast<size_t>(idx) >= n_user) {
          return fail("capture " + id + " out of range");
        }
        *r = id;
        return true;
      }
      for (const Builtin& bi : kBuiltins) {
        if (id == bi.name) {
          skip();
          if (s[pos] != '(') return fail("expected '(' after " + id);
          ++pos;
          std::string args;
          for (int a = 0; a < bi.arity; ++a) {
            std::string e;
            if (!additive(&e)) return false;
            skip();
            if (a + 1 < bi.arity) {
              if (s[pos] != ',') return fail(id + " takes " + std::to_string(bi.arity) + " arguments");
              ++pos;
              args += e + ", ";
            } else {
              args += e;
            }
          }
          if (s[pos] != ')') return fail("expected ')' closing " + id);
          ++pos;
          *r = id + "(" + args + ")";
          return true;
        }
      }
      return fail("unknown identifier '" + id + "'");
    }
    return fail("unexpected character");
  }
  bool multiplicative(std::string* r) {
    if (!primary(r)) return false;
    for (;;) {
      skip();
      const char c = s[pos];
      if (c != '*' && c != '/') return true;
      ++pos;
      std::string b;
      if (!primary(&b)) return false;
      *r = "(" + *r + " " + c + " " + b + ")";
    }
  }
  bool additive(std::string* r) {
    if (!multiplicative(r)) return false;
    for (;;) {
      skip();
      const char c = s[pos];
      if (c != '+' && c != '-') return true;
      ++pos;
      std::string b;
      if (!multiplicative(&b)) return false;
      *r = "(" + *r + " " + c + " " + b + ")";
    }
  }
};

}  // namespace

bool canonicalize(const char* src, int max_operands, const std::vector<float>& user_captures,
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
  Parser p{src, 0, max_operands, user_captures.size(), out, {}, 0};
  std::string r;
  bool ok = p.additive(&r);
  if (ok) {
    p.skip();
    if (src[p.pos] != '\0') ok = p.fail("trailing characters");
  }
  if (!ok) {
    if (err) *err = p.err;
    return false;
  }
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
