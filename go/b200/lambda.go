package b200

import (
	"fmt"
	"strconv"
	"strings"

	"tcacomp/internal/ir"
)

// lambdaPrinter prints one lambda body as the C expression text the C ABI
// takes: the same walk the reference's emitter makes over a pure value tree
// (internal/cg/cxx/expr.go:14-101), with the operator spellings of
// internal/cg/cxx/naming.go:126-183 and the builtin names of :188-198.
// Lambda-bound parameters become p0, p1, ... in the order the lambda declares
// them; a scalar kernel parameter becomes a capture slot c0, c1, ..., numbered
// by first appearance and remembered in Captures.
type lambdaPrinter struct {
	params   map[ir.Node]int // lambda-bound InputParam -> position
	Captures []string        // scalar parameter name of each capture slot
}

func newLambdaPrinter(lambda ir.Node, first int) *lambdaPrinter {
	ops := ir.OperandsOf(lambda) // (param declarations..., body): internal/ir/node_lambda.go:60-66
	lp := &lambdaPrinter{params: map[ir.Node]int{}}
	for i, p := range ops[:len(ops)-1] {
		lp.params[p] = first + i
	}
	return lp
}

func lambdaBody(lambda ir.Node) ir.Node {
	ops := ir.OperandsOf(lambda)
	return ops[len(ops)-1]
}

func (lp *lambdaPrinter) capture(name string) string {
	for i, c := range lp.Captures {
		if c == name {
			return "c" + strconv.Itoa(i)
		}
	}
	lp.Captures = append(lp.Captures, name)
	return "c" + strconv.Itoa(len(lp.Captures)-1)
}

var elemCxx = map[ir.ElemType]string{ // internal/cg/cxx/naming.go:21-46, the types this library moves
	ir.TF32: "float", ir.TBF16: "__nv_bfloat16", ir.TI32: "int32_t", ir.TU32: "uint32_t",
}

func (lp *lambdaPrinter) print(n ir.Node) (string, error) {
	switch n.KindOf() {
	case ir.KindConst:
		v, ok := ir.ConstValueOf(n)
		nt, isNum := ir.ConstTypeOf(n).(*ir.NumericType)
		if !ok || !isNum {
			return "", fmt.Errorf("b200: const %d carries no typed value", n.BasePtr().ID())
		}
		switch nt.Elem() { // literal forms: internal/cg/cxx/naming.go:90-122
		case ir.TF32:
			lit := strconv.FormatFloat(v, 'g', -1, 32)
			if !strings.ContainsAny(lit, ".eE") {
				lit += ".0"
			}
			return lit + "f", nil
		case ir.TU32:
			return strconv.FormatUint(uint64(v), 10) + "u", nil
		case ir.TI32:
			if v < 0 {
				return "(-" + strconv.FormatInt(-int64(v), 10) + ")", nil
			}
			return strconv.FormatInt(int64(v), 10), nil
		case ir.TBool:
			if v != 0 {
				return "true", nil
			}
			return "false", nil
		}
		return "", fmt.Errorf("b200: a %s constant has no literal form", nt.Elem())
	case ir.KindParam: // a reference to an InputParam: lambda-bound or a scalar kernel parameter
		def := ir.OperandsOf(n)[0]
		if i, ok := lp.params[def]; ok {
			return "p" + strconv.Itoa(i), nil
		}
		if role, ok := ir.RoleOf(def); ok && role == ir.RoleScalar {
			return lp.capture(ir.InputParamNameOf(def)), nil
		}
		return "", fmt.Errorf("b200: param %s is neither bound by this lambda nor a scalar parameter", ir.InputParamNameOf(def))
	case ir.KindBinOp:
		op, _ := ir.BinOpCodeOf(n)
		ops := ir.OperandsOf(n)
		l, err := lp.print(ops[0]) // left before right: capture slots are numbered in print order
		if err != nil {
			return "", err
		}
		r, err := lp.print(ops[1])
		if err != nil {
			return "", err
		}
		return "(" + l + " " + op.String() + " " + r + ")", nil
	case ir.KindUnaryOp:
		op, _ := ir.UnaryOpCodeOf(n)
		x, err := lp.print(ir.OperandsOf(n)[0])
		if err != nil {
			return "", err
		}
		if op == ir.UnaryOpPos {
			return x, nil
		}
		return "(" + op.String() + x + ")", nil
	case ir.KindSelect: // internal/cg/cxx/expr.go:38-56
		ops := ir.OperandsOf(n)
		parts := make([]string, 3)
		for i := range parts {
			s, err := lp.print(ops[i])
			if err != nil {
				return "", err
			}
			parts[i] = s
		}
		return "(" + parts[0] + " ? " + parts[1] + " : " + parts[2] + ")", nil
	case ir.KindCast: // internal/cg/cxx/expr.go:57-66
		nt, ok := ir.CastTypeOf(n).(*ir.NumericType)
		if !ok {
			return "", fmt.Errorf("b200: cast %d carries no numeric type", n.BasePtr().ID())
		}
		ts, ok := elemCxx[nt.Elem()]
		if !ok {
			return "", fmt.Errorf("b200: a cast to %s has no kernel in the library (f32, bf16, i32, u32)", nt.Elem())
		}
		x, err := lp.print(ir.OperandsOf(n)[0])
		if err != nil {
			return "", err
		}
		return "static_cast<" + ts + ">(" + x + ")", nil
	case ir.KindCall: // builtins verbatim (internal/cg/cxx/naming.go:188-198); umin / umax are CUDA's
		args := make([]string, 0, 3)
		for _, a := range ir.OperandsOf(n) {
			s, err := lp.print(a)
			if err != nil {
				return "", err
			}
			args = append(args, s)
		}
		return ir.CallNameOf(n) + "(" + strings.Join(args, ", ") + ")", nil
	}
	return "", fmt.Errorf("b200: node %d (%s) is not a scalar expression", n.BasePtr().ID(), n.KindOf())
}

// PrintLambda prints the body of `lambda` (a KindLambda node: ir.LambdaOf of
// a Map or Reduce). first shifts the parameter numbering (0 everywhere: a
// piped map's parameter 0 is the piped value). It returns the text and the
// scalar parameter behind each capture slot.
func PrintLambda(lambda ir.Node, captures []string) (string, []string, error) {
	lp := newLambdaPrinter(lambda, 0)
	lp.Captures = captures
	s, err := lp.print(lambdaBody(lambda))
	return s, lp.Captures, err
}
