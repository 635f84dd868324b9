// Package b200 is the reference-side shim over libtcab.so: it classifies the
// statements of a graph built with the UNCHANGED pkg builder
// (pkg/builder.go, pkg/chain.go, pkg/expr.go) and launches each one through
// the C ABI of include/tcab.h, in place of compile -> cxx.Emit -> nvcc ->
// <Name>Launch (internal/compiler/compiler.go:26-41,
// internal/cg/cxx/emit.go:85-190, internal/cg/cxx/launch.go:23-156).
//
// Placement: the package imports tcacomp/internal/ir, so it lives inside the
// reference's module, e.g. as internal/b200 (copy this directory there and
// point the cgo flags in tcab.go at the installed include/ and lib/).
//
// Status: written against the accessors the reference's own emitter uses
// (ir.OperandsOf, ir.LambdaOf, ir.AsOf, ir.ReduceInitOf, ir.BinOpCodeOf,
// ir.UnaryOpCodeOf, ir.CallNameOf, ir.ConstValueOf, ir.ConstTypeOf,
// ir.CastTypeOf, ir.RoleOf, ir.InputParamNameOf, ir.InputParamTypeOf) and
// NOT compiled: the image this library was built in has no Go toolchain, and
// neither has the GPU box it was measured on. The same classification, over
// a C++ mirror of the builder, is compiled and tested in
// tcacomp_b200/csrc/host/pkg_launch.cpp (tests/cpp/host_tests.cpp,
// tests/test_tca_text.py); classify_test.go states the same expectations for
// this package.
package b200
