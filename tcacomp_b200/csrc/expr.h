// expr.h -- the scalar-lambda expressions that cross the C ABI.
//
// A lambda arrives as a C expression in the reference's operator and builtin
// vocabulary (internal/cg/cxx/naming.go:126-198, internal/ir/builtins.go:25-39)
// and is TYPED the way the reference's builder types it (pkg/expr.go:137-176,
// 185-203, 271): operands p0.. carry their tensor's element type, captures
// c0.. are f32, floating literals are f32, decimal integers i32, integers with
// a trailing u are u32, true / false are bool; binary operators take two
// operands of ONE type, with no implicit promotion; comparisons give bool;
// && || ! take bool; % & | ^ << >> ~ take one integer type; cond ? a : b takes a
// bool and two branches of one type; a conversion is always explicit,
// static_cast<T>(x) between arithmetic types (internal/ir/types.go:60-62), also
// accepted in the short spellings f32(x), bf16(x), i32(x), u32(x). bf16 is a
// storage type (design/syntax-design.md:601-607): a bf16 value can be converted
// and selected, nothing else.
//
// canonicalize() validates the text (nothing else may reach a compiler), prints
// it fully parenthesised, and LIFTS every f32 literal into a capture slot --
// equal literals share a slot -- so that one compiled kernel serves every
// choice of constants:
//     "(0.5f*p0 + 0.25f) * (0.5f*p0 + 0.25f)"  ->  "(((c0 * p0) + c1) * ((c0 * p0) + c1))", {0.5, 0.25}
// Integer and bool literals stay in the text (they are part of the kernel).
#pragma once

#include <string>
#include <vector>

namespace tcab {

enum ElemT { kF32 = 0, kBF16 = 1, kI32 = 2, kU32 = 3, kBool = 4 };  // the first four match tcab_dtype
const char* elem_name(ElemT t);        // "f32", "bf16", ...
const char* elem_cxx(ElemT t);         // the C++ spelling the reference emits (internal/cg/cxx/naming.go:21-46)

struct CanonExpr {
  std::string text;             // canonical spelling over p*, c*
  std::vector<float> captures;  // values of c0.. in the canonical text (numbered by first appearance)
  int n_operands = 0;           // highest p index used + 1
  ElemT type = kF32;            // type of the whole expression
};

// Returns false and fills `err` on a syntax error, a type error, an unknown identifier, an
// operand index >= max_operands or a capture index >= user_captures.size().
// operand_types: max_operands entries, or null when every operand is f32.
bool canonicalize(const char* src, int max_operands, const ElemT* operand_types,
                  const std::vector<float>& user_captures, CanonExpr* out, std::string* err);

}  // namespace tcab
