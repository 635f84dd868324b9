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
//   expr        ::= cond '?' expr ':' expr | the binary operators || && | ^ & == != < <= > >= << >> + - * / % with C
//                   precedence | unary - + ! ~ | calls of the builtins | casts elem '(' expr ')' | literals
//                   (1.5f, 3, 8u, true, false, inf_f32) | names (lambda parameters, captured scalar parameters)
//
// A kernel may bind several lets (design/syntax-design.md 5.1, lowering table: a `let` that is not the returned
// one becomes a Local that its chain stores into and later chains bind as an operand, pkg/builder.go:224). An
// operand may bind a subset of the iteration's dimvars (m[i] inside an (i, j) iteration). One construct goes
// beyond the reference's v0: a let whose chain is a map alone (the reference requires a reduction before a
// store, pkg/chain.go:433-438) is lowered through the added rung of pkg_ext.h, because the kernel library has
// the map-only operator; it is what the last statement of a softmax or a layer-norm needs.
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

// A module spread over several files (the reference's loader reads them from disk, internal/syntax/module.go:
// 3-31; here the host hands over the texts, this library does no file I/O): `root` names the entry file among
// `files`; @include paths are resolved relative to the including file, may not be absolute nor leave its
// directory, a file reached twice merges once, a cycle is an error; an included file's kernels land after the
// including file's own. Diagnostics of included files are prefixed with their path.
struct SourceFile {
  std::string path, text;
};
Result<std::vector<ParsedKernel>> ParseModuleFiles(const std::vector<SourceFile>& files, const std::string& root);

}  // namespace pkg
}  // namespace tcab
