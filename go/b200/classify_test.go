package b200

import (
	"testing"

	"tcacomp/internal/ir"
	"tcacomp/pkg"
)

// The chain of pkg/oracle_test.go:17-63 (matmul_scale) built through the
// unchanged rungs classifies as a contraction with a piped scale; the
// expectations equal those of the C++ mirror (tests/cpp/host_tests.cpp).
func TestMatmulScaleClassifiesAsContraction(t *testing.T) {
	b := pkg.NewBuilder("matmul_scale")
	m, k, n := b.Dim("m", 0), b.Dim("k", 0), b.Dim("n", 0)
	lhs := b.Tensor("lhs", ir.TF32, m, n)
	rhs := b.Tensor("rhs", ir.TF32, n, k)
	out := b.Tensor("output", ir.TF32, m, k)
	scale := b.ScalarParam("scale", ir.TF32)
	root, err := b.Stmt().Iter(m, k, n).Map([]pkg.Operand{pkg.At(lhs, m, n), pkg.At(rhs, n, k)},
		func(l, r pkg.Expr) pkg.Expr { return b.Mul(l, r) })
	if err != nil {
		t.Fatal(err)
	}
	ar, err := root.As(m, k, n).Reduce(b.Float32(0), func(acc, v pkg.Expr) pkg.Expr { return b.Add(acc, v) })
	if err != nil {
		t.Fatal(err)
	}
	am, err := ar.Map(nil, func(v pkg.Expr) pkg.Expr { return b.Mul(v, scale) })
	if err != nil {
		t.Fatal(err)
	}
	if _, err := am.As(m, k).Store(out, m, k); err != nil {
		t.Fatal(err)
	}
	g, err := b.Build()
	if err != nil {
		t.Fatal(err)
	}
	plans, err := PlanGraph(g)
	if err != nil || len(plans) != 1 {
		t.Fatalf("plans %v err %v", plans, err)
	}
	p := plans[0]
	if p.Kind != ChainContract || p.RhsIsNK || p.Map != "(p0 * p1)" || p.Combine != "(p0 + p1)" || p.Post != "(p0 * c0)" ||
		len(p.Captures) != 1 || p.Captures[0] != "scale" || p.Out != "output" {
		t.Fatalf("unexpected plan %+v", p)
	}
}

// The first benchmark configuration: y[i] = sum_j (0.5 x[i][j] + 0.25)^2.
func TestAffineSquareRowSumClassifiesAsChainReduce(t *testing.T) {
	b := pkg.NewBuilder("c1")
	i, j := b.Dim("i", 0), b.Dim("j", 0)
	x := b.Tensor("x", ir.TF32, i, j)
	y := b.Tensor("y", ir.TF32, i)
	root, err := b.Stmt().Iter(i, j).Map([]pkg.Operand{pkg.At(x, i, j)}, func(v pkg.Expr) pkg.Expr {
		a := b.Add(b.Mul(b.Float32(0.5), v), b.Float32(0.25))
		return b.Mul(a, a)
	})
	if err != nil {
		t.Fatal(err)
	}
	ar, err := root.As(i, j).Reduce(b.Float32(0), func(acc, v pkg.Expr) pkg.Expr { return b.Add(acc, v) })
	if err != nil {
		t.Fatal(err)
	}
	if _, err := ar.Store(y, i); err != nil {
		t.Fatal(err)
	}
	g, err := b.Build()
	if err != nil {
		t.Fatal(err)
	}
	plans, err := PlanGraph(g)
	if err != nil || len(plans) != 1 {
		t.Fatalf("plans %v err %v", plans, err)
	}
	p := plans[0]
	if p.Kind != ChainReduce || p.ReduceAxis != 1 || p.Map != "(((0.5f * p0) + 0.25f) * ((0.5f * p0) + 0.25f))" || p.Init != 0 {
		t.Fatalf("unexpected plan %+v", p)
	}
}

// Select and comparisons print the way the emitter prints them
// (internal/cg/cxx/expr.go:38-56, internal/cg/cxx/naming.go:126-183).
func TestSelectPrintsAsConditional(t *testing.T) {
	b := pkg.NewBuilder("relu")
	i, j := b.Dim("i", 0), b.Dim("j", 0)
	x := b.Tensor("x", ir.TF32, i, j)
	y := b.Tensor("y", ir.TF32, i)
	root, _ := b.Stmt().Iter(i, j).Map([]pkg.Operand{pkg.At(x, i, j)}, func(v pkg.Expr) pkg.Expr {
		return pkg.Select(b.Gt(v, b.Float32(0)), v, b.Float32(0))
	})
	ar, _ := root.As(i, j).Reduce(b.Float32(0), func(acc, v pkg.Expr) pkg.Expr { return b.Add(acc, v) })
	if _, err := ar.Store(y, i); err != nil {
		t.Fatal(err)
	}
	g, err := b.Build()
	if err != nil {
		t.Fatal(err)
	}
	plans, err := PlanGraph(g)
	if err != nil || plans[0].Map != "((p0 > 0.0f) ? p0 : 0.0f)" {
		t.Fatalf("plans %+v err %v", plans, err)
	}
}
