// tca_syntax.h -- the .tca text frontend over the C++ builder mirror.
//
// The reference's frontend (internal/syntax: lexer, parser, semacheck, build) turns a kernel written in
// its text DSL into calls on the pkg rungs (internal/syntax/build/build.go:27-36). This is the same step
// for the grammar of design/syntax-design.md section 2, restricted to what this path evaluates:
//
//   module      ::= { '@include' string ';' | '@runtime' '(' keyed ')' ';' | kernel }
//   kernel      ::= { '@' ident '(' keyed ')' } 'kernel' ident '(' params ')' '->' type '{' stmts '}'
//   param       ::= ident ':' ( 'tensor' '<' 'dtype' '=' elem ',' 'shape' '=' '[' dims ']' '>' | elem )
//   stmt        ::= 'dimvar' [ '(' ] idents [ ')' ] ';' | 'let' ident [ ':' type ] '=' chain ';' | 'return' ident ';'
//   chain       ::= stage { '|' stage }
//   map stage   ::= 'map' 'on' '(' bindings ')' [ 'as' '(' idents ')' ] [ '[' captures ']' ] '(' params ')' [ '->' elem ] ':' expr
//   reduce      ::= 'reduce' '(' 'init' '=' expr ')' 'on' '(' acc ':' elem ',' ( '%0' | ident ) [ ':' elem ] ')'
//                   [ 'as' '(' idents ')' ] '->' elem ':' expr
//   expr        ::= + - * / , unary -, calls of the fp32 builtins, casts elem '(' expr ')', literals
//                   (1.5f, 3, 8u, inf_f32), names (lambda parameters, captured scalar parameters)
//
// Comparisons, ?:, bit operators and bool are parsed by the reference but have no kernel class here;
// they are reported as unsupported. One kernel = one let chain ending in `return <that let>`.
// Trailing commas are accepted in every list; // and /* */ comments are skipped.
#pragma once

#include <string>
#include <vector>

#include "pkg.h"

namespace tcab {
namespace pkg {

struct ParsedKernel {
  std::string name;      // kernel identifier
  std::string cxx_name;  // @name(cxx="...") if present, else the identifier
  std::string output;    // name of the returned let: the output tensor's name in the graph
  Graph graph;
};

// Parses a module and lowers every kernel through the builder rungs. On failure err carries
// "line:col: message" like the reference's diagnostics.
Result<std::vector<ParsedKernel>> ParseModule(const std::string& text);

}  // namespace pkg
}  // namespace tcab
