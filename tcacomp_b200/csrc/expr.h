// expr.h -- the scalar-lambda expressions that cross the C ABI.
//
// A lambda arrives as a C expression in the reference's operator and builtin
// vocabulary (internal/cg/cxx/naming.go:126-198, internal/ir/builtins.go:25-39):
// operands p0.., scalar captures c0.., fp32 literals, + - * /, unary minus and
// the fp32 builtins. canonicalize() validates it (nothing else may reach a
// compiler), prints it fully parenthesised, and LIFTS every literal into a
// capture slot -- equal literals share a slot -- so that one compiled kernel
// serves every choice of constants:
//     "(0.5f*p0 + 0.25f) * (0.5f*p0 + 0.25f)"  ->  "(((c0 * p0) + c1) * ((c0 * p0) + c1))", {0.5, 0.25}
#pragma once

#include <string>
#include <vector>

namespace tcab {

struct CanonExpr {
  std::string text;             // canonical spelling over p*, c*
  std::vector<float> captures;  // values of c0.. in the canonical text (numbered by first appearance)
  int n_operands = 0;           // highest p index used + 1
};

// Returns false and fills `err` on a syntax error, an unknown identifier, an
// operand index >= max_operands or a capture index >= user_captures.size().
bool canonicalize(const char* src, int max_operands, const std::vector<float>& user_captures,
                  CanonExpr* out, std::string* err);

}  // namespace tcab
