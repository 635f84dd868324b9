package b200

import (
	"fmt"

	"tcacomp/internal/ir"
)

// Kind names the entry point of include/tcab.h a statement lowers to.
type Kind int

const (
	ChainReduce Kind = iota
	ChainContract
	GemmBiasAct
	MapOnly
)

// Plan is what one stored statement lowers to: the entry point, the lambdas as
// C text, and the tensors by name in operand order. It is the Go twin of
// tcab::pkg::Plan (tcacomp_b200/csrc/host/pkg.h).
type Plan struct {
	Kind                     Kind
	Map, Combine, Post       string
	Init                     float32
	Captures                 []string // scalar parameter of capture slot i
	Inputs                   []string // tensor names, in operand order
	Indexing                 []int    // per operand: 0 every axis, 1 one value per row, 2 one row shared by all rows, 3 one value per output cell (middle-axis reductions)
	ReduceAxis               uint32
	RhsIsNK                  bool
	A, B, Bias               string
	Relu                     bool
	Out                      string
}

// operand is one structural tensor access of a map: the MemLoad's tensor
// InputParam and the dim InputParams that subscript it (internal/ir/node_memory.go:
// ops = [src, axes...]).
type operand struct {
	name string
	elem ir.ElemType
	axes []string
}

func loadOf(n ir.Node) (operand, error) {
	if n.KindOf() != ir.KindMemLoad {
		return operand{}, fmt.Errorf("b200: map operand %d is a %s, not a tensor access", n.BasePtr().ID(), n.KindOf())
	}
	ops := ir.OperandsOf(n)
	t, _ := ir.InputParamTypeOf(ops[0])
	nt, ok := t.(*ir.NumericType)
	if !ok {
		return operand{}, fmt.Errorf("b200: tensor %s carries no numeric type", ir.InputParamNameOf(ops[0]))
	}
	o := operand{name: ir.InputParamNameOf(ops[0]), elem: nt.Elem()}
	for _, a := range ops[1:] {
		o.axes = append(o.axes, ir.InputParamNameOf(a))
	}
	return o, nil
}

func names(nodes []ir.Node) []string {
	out := make([]string, len(nodes))
	for i, n := range nodes {
		out[i] = ir.InputParamNameOf(n)
	}
	return out
}

func same(a, b []string) bool {
	if len(a) != len(b) {
		return false
	}
	for i := range a {
		if a[i] != b[i] {
			return false
		}
	}
	return true
}

func movable(e ir.ElemType) bool { return e == ir.TF32 || e == ir.TBF16 || e == ir.TI32 || e == ir.TU32 }

// valueOperands returns the tensor accesses a Map binds: its value operands are
// IterClusterProject bridges into the iteration cluster's input list
// (internal/ir/node_iterfmt.go:40-57, internal/ir/node_loop.go:74-83); a piped
// map's first value operand is the previous stage instead.
func valueOperands(m ir.Node) (loads []ir.Node, piped ir.Node) {
	ops := ir.OperandsOf(m)
	for _, op := range ops {
		if op == nil {
			continue
		}
		switch op.KindOf() {
		case ir.KindAs, ir.KindLambda:
		case ir.KindIterClusterProject:
			idx, _ := ir.IterClusterProjectIndex(op)
			cluster := ir.OperandsOf(op)[0]
			loads = append(loads, ir.ClusterInputs(cluster)[idx])
		case ir.KindReduce, ir.KindMap:
			piped = op
		case ir.KindMemLoad:
			loads = append(loads, op)
		}
	}
	return loads, piped
}

// Classify matches one statement -- memstore(target[axes], value), ops = (value,
// tensor, axes...) as internal/ir/node_memory.go:113-118 builds it -- to an
// entry point. The chain behind `value` is root map [| reduce [| piped map]].
func Classify(store ir.Node) (Plan, error) {
	var p Plan
	if store.KindOf() != ir.KindMemStore {
		return p, fmt.Errorf("b200: statement root is a %s, not a store", store.KindOf())
	}
	sops := ir.OperandsOf(store)
	value, target := sops[0], sops[1]
	p.Out = ir.InputParamNameOf(target)
	outAxes := names(sops[2:])

	var post, reduce, root ir.Node
	cur := value
	if cur.KindOf() == ir.KindMap {
		if _, piped := valueOperands(cur); piped != nil {
			post, cur = cur, piped
		}
	}
	if cur.KindOf() == ir.KindReduce {
		reduce = cur
		cur = ir.OperandsOf(cur)[0] // (piped, KeyedAttribute init, lambda): internal/ir/node_lambda.go:99-109
	}
	if cur.KindOf() == ir.KindReduce {
		return p, fmt.Errorf("b200: several reductions in one chain; the kernel library reduces one axis per launch")
	}
	if cur.KindOf() != ir.KindMap {
		return p, fmt.Errorf("b200: the chain does not begin with a root map")
	}
	root = cur
	loads, _ := valueOperands(root)
	if len(loads) == 0 {
		return p, fmt.Errorf("b200: a map without tensor operands has no kernel class")
	}
	as := names(ir.OperandsOf(ir.AsOf(root)))
	ops := make([]operand, len(loads))
	var full *operand
	for i, l := range loads {
		o, err := loadOf(l)
		if err != nil {
			return p, err
		}
		if !movable(o.elem) {
			return p, fmt.Errorf("b200: operand %s is %s; the kernels move f32, bf16, i32 and u32", o.name, o.elem)
		}
		ops[i] = o
		if full == nil && len(o.axes) == len(as) {
			full = &ops[i]
		}
		p.Inputs = append(p.Inputs, o.name)
	}

	var err error
	if p.Map, p.Captures, err = PrintLambda(ir.LambdaOf(root), nil); err != nil {
		return p, err
	}
	if reduce != nil {
		init := ir.ReduceInitOf(reduce)
		v, ok := ir.ConstValueOf(init)
		if !ok {
			return p, fmt.Errorf("b200: the reduction's init must be a literal")
		}
		p.Init = float32(v)
		var none []string
		if p.Combine, none, err = PrintLambda(ir.LambdaOf(reduce), nil); err != nil {
			return p, err
		}
		if len(none) != 0 {
			return p, fmt.Errorf("b200: a combiner may not capture scalar parameters")
		}
	}
	if post != nil {
		if loads, _ := valueOperands(post); len(loads) != 0 {
			return p, fmt.Errorf("b200: a piped map with tensor operands is only covered by the tensor-core contraction class")
		}
		if p.Post, p.Captures, err = PrintLambda(ir.LambdaOf(post), p.Captures); err != nil {
			return p, err
		}
	}

	// contraction: lhs[m,k] with rhs[k,n] or rhs[n,k], as (m, n, k), out[m,n]
	if reduce != nil && len(ops) == 2 && len(as) == 3 && len(ops[0].axes) == 2 && len(ops[1].axes) == 2 {
		m, n, k := as[0], as[1], as[2]
		kn := same(ops[1].axes, []string{k, n})
		nk := same(ops[1].axes, []string{n, k})
		if same(ops[0].axes, []string{m, k}) && (kn || nk) && same(outAxes, []string{m, n}) {
			p.Kind, p.RhsIsNK = ChainContract, nk
			return p, nil
		}
	}
	if full == nil {
		return p, fmt.Errorf("b200: no operand carries every iteration axis; a chain needs one operand that fixes the layout")
	}
	axes := full.axes
	// under a reduction of an axis that is not the innermost: all axes but the reduced one (one value per output cell)
	var cellAxes []string
	if reduce != nil && len(as) > 0 && len(axes) > 1 && axes[len(axes)-1] != as[len(as)-1] {
		for _, a := range axes {
			if a != as[len(as)-1] {
				cellAxes = append(cellAxes, a)
			}
		}
	}
	for _, o := range ops {
		switch {
		case same(o.axes, axes):
			p.Indexing = append(p.Indexing, 0)
		case cellAxes != nil && same(o.axes, cellAxes):
			p.Indexing = append(p.Indexing, 3)
		case cellAxes != nil:
			return p, fmt.Errorf("b200: operand %s: under a reduction of a middle axis an operand carries every axis or all but the reduced one", o.name)
		case len(axes) > 1 && same(o.axes, axes[:len(axes)-1]):
			p.Indexing = append(p.Indexing, 1)
		case len(axes) > 1 && same(o.axes, axes[len(axes)-1:]):
			p.Indexing = append(p.Indexing, 2)
		default:
			return p, fmt.Errorf("b200: operand %s is indexed by an axis subset no kernel class takes", o.name)
		}
	}
	if reduce == nil { // a map alone: stored through an added rung, never by the reference's own rungs (pkg/chain.go:433-438)
		if !same(as, axes) || !same(outAxes, axes) {
			return p, fmt.Errorf("b200: a stored map keeps the operands' axis order")
		}
		p.Kind = MapOnly
		return p, nil
	}
	red := as[len(as)-1]
	pos := -1
	var rest []string
	for i, a := range axes {
		if a == red {
			pos = i
		} else {
			rest = append(rest, a)
		}
	}
	if pos < 0 || !same(rest, as[:len(as)-1]) || !same(outAxes, rest) {
		return p, fmt.Errorf("b200: the output must keep the operands' axis order minus the reduced axis @%s", red)
	}
	p.Kind, p.ReduceAxis = ChainReduce, uint32(pos)
	return p, nil
}

// PlanGraph classifies every store statement of g in program order. (The
// statement groups that spell a whole row softmax or layer-norm are recognised
// on the finished plans exactly as tcab::pkg::PlanGraph does; that pass works on
// the printed lambdas and is not repeated here.)
func PlanGraph(g *ir.Graph) ([]Plan, error) {
	var plans []Plan
	for s := g.Block().First(); s != nil; s = s.Next() {
		rhs := s.RHS()
		if rhs == nil || rhs.KindOf() != ir.KindMemStore {
			continue // the return statement
		}
		p, err := Classify(rhs)
		if err != nil {
			return nil, fmt.Errorf("statement #%d: %w", s.ID(), err)
		}
		plans = append(plans, p)
	}
	return plans, nil
}
