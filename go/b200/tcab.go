package b200

/*
#cgo CFLAGS: -I${SRCDIR}/../../third_party/tcab/include
#cgo LDFLAGS: -L${SRCDIR}/../../third_party/tcab/lib -ltcab
#include <stdlib.h>
#include "tcab.h"
*/
import "C"

import (
	"errors"
	"runtime"
	"unsafe"
)

// Element types of include/tcab.h (tcab_dtype).
const (
	F32  = int32(C.TCAB_F32)
	BF16 = int32(C.TCAB_BF16)
	I32  = int32(C.TCAB_I32)
	U32  = int32(C.TCAB_U32)
)

// Tensor mirrors tca::Tensor<T,R> (runtime/tca/tensor.h:16-40): a non-owning
// view of row-major contiguous DEVICE memory. The caller owns the memory.
type Tensor struct {
	Data  unsafe.Pointer
	DType int32
	Dims  []uint32 // slowest first, rank 1..4
}

func (t Tensor) c() C.tcab_tensor {
	var ct C.tcab_tensor
	ct.data = t.Data
	ct.dtype = C.int32_t(t.DType)
	ct.rank = C.uint32_t(len(t.Dims))
	for i, d := range t.Dims {
		ct.dims[i] = C.uint32_t(d)
	}
	return ct
}

// Chain is tcab_chain: the lambdas of a map | reduce | map statement as C
// expression text (what PrintLambda produces), the reduction's init and the
// values of the captured scalar parameters, slot by slot.
type Chain struct {
	Map, Combine, Post string // Post == "": the reduction is stored as it is
	Init               float32
	Captures           []float32
}

// withChain builds the C struct and frees its strings after f returns.
func withChain(ch Chain, f func(*C.tcab_chain) C.int) C.int {
	var cc C.tcab_chain
	cc.map_expr = C.CString(ch.Map)
	defer C.free(unsafe.Pointer(cc.map_expr))
	if ch.Combine != "" {
		cc.combine_expr = C.CString(ch.Combine)
		defer C.free(unsafe.Pointer(cc.combine_expr))
	}
	if ch.Post != "" {
		cc.post_expr = C.CString(ch.Post)
		defer C.free(unsafe.Pointer(cc.post_expr))
	}
	cc.init = C.float(ch.Init)
	cc.n_captures = C.uint32_t(len(ch.Captures))
	for i, v := range ch.Captures {
		cc.captures[i] = C.float(v)
	}
	return f(&cc)
}

// call runs one entry point on a locked OS thread: the library's error text
// is thread-local, so the status and its message must be read on one thread.
func call(f func() C.int) error {
	runtime.LockOSThread()
	defer runtime.UnlockOSThread()
	if rc := f(); rc != C.TCAB_OK {
		return errors.New(C.GoString(C.tcab_last_error()))
	}
	return nil
}

func cTensors(ts []Tensor) []C.tcab_tensor {
	out := make([]C.tcab_tensor, len(ts))
	for i, t := range ts {
		out[i] = t.c()
	}
	return out
}

// ChainReduce launches out = post(fold_k map(ins...)) on stream (a
// cudaStream_t), asynchronously. tcab_chain_reduce.
func ChainReduce(ch Chain, ins []Tensor, reduceAxis uint32, out Tensor, stream unsafe.Pointer) error {
	cin, cout := cTensors(ins), out.c()
	return call(func() C.int {
		return withChain(ch, func(cc *C.tcab_chain) C.int {
			return C.tcab_chain_reduce(cc, &cin[0], C.uint32_t(len(ins)), C.uint32_t(reduceAxis), &cout, stream)
		})
	})
}

// ChainReduceBatched hands several problems of one shape to one launch.
// problems[b] are the operands of problem b. tcab_chain_reduce_batched.
func ChainReduceBatched(ch Chain, problems [][]Tensor, outs []Tensor, stream unsafe.Pointer) error {
	nIns := len(problems[0])
	flat := make([]C.tcab_tensor, 0, len(problems)*nIns)
	for _, p := range problems {
		flat = append(flat, cTensors(p)...)
	}
	couts := cTensors(outs)
	return call(func() C.int {
		return withChain(ch, func(cc *C.tcab_chain) C.int {
			return C.tcab_chain_reduce_batched(cc, &flat[0], C.uint32_t(nIns), C.uint32_t(len(problems)), &couts[0], stream)
		})
	})
}

// Map launches the map-only chain out[...] = map(ins[0][...], ...). tcab_map.
func Map(ch Chain, ins []Tensor, out Tensor, stream unsafe.Pointer) error {
	cin, cout := cTensors(ins), out.c()
	return call(func() C.int {
		return withChain(ch, func(cc *C.tcab_chain) C.int {
			return C.tcab_map(cc, &cin[0], C.uint32_t(len(ins)), &cout, stream)
		})
	})
}

// ChainContract launches out[m,n] = post(fold_k map(lhs[m,k], rhs[k,n])) (rhs[n,k]
// with rhsIsNK). tcab_chain_contract.
func ChainContract(ch Chain, lhs, rhs Tensor, rhsIsNK bool, out Tensor, stream unsafe.Pointer) error {
	cl, cr, co := lhs.c(), rhs.c(), out.c()
	nk := C.int(0)
	if rhsIsNK {
		nk = 1
	}
	return call(func() C.int {
		return withChain(ch, func(cc *C.tcab_chain) C.int {
			return C.tcab_chain_contract(cc, &cl, &cr, nk, &co, stream)
		})
	})
}

// ReduceOuter reduces t[b,k,c] over k in one pass; nil outputs are skipped.
func ReduceOuter(t Tensor, sum, max, argmax *Tensor, stream unsafe.Pointer) error {
	ct := t.c()
	opt := func(p *Tensor) *C.tcab_tensor {
		if p == nil {
			return nil
		}
		v := p.c()
		return &v
	}
	cs, cm, ca := opt(sum), opt(max), opt(argmax)
	return call(func() C.int { return C.tcab_reduce_outer(&ct, cs, cm, ca, stream) })
}

func SoftmaxRows(x, y Tensor, stream unsafe.Pointer) error {
	cx, cy := x.c(), y.c()
	return call(func() C.int { return C.tcab_softmax_rows(&cx, &cy, stream) })
}

func LayernormRows(x, gamma, beta Tensor, eps float32, y Tensor, stream unsafe.Pointer) error {
	cx, cg, cb, cy := x.c(), gamma.c(), beta.c(), y.c()
	return call(func() C.int { return C.tcab_layernorm_rows(&cx, &cg, &cb, C.float(eps), &cy, stream) })
}

func GemmBiasAct(a, b Tensor, bias *Tensor, relu bool, c Tensor, stream unsafe.Pointer) error {
	ca, cb, cc := a.c(), b.c(), c.c()
	var pb *C.tcab_tensor
	if bias != nil {
		t := bias.c()
		pb = &t
	}
	act := C.int(C.TCAB_ACT_NONE)
	if relu {
		act = C.TCAB_ACT_RELU
	}
	return call(func() C.int { return C.tcab_gemm_bias_act(&ca, &cb, pb, act, &cc, stream) })
}

// Prepare compiles now what the first launch of a chain without an
// ahead-of-time kernel would compile later (tcab_chain_prepare); use is one of
// C.TCAB_USE_REDUCE, _CONTRACT, _MAP, _REDUCE_BATCHED. Not during a stream capture.
func Prepare(ch Chain, inDTypes []int32, use int, outDType int32) error {
	types := make([]C.int32_t, len(inDTypes))
	for i, t := range inDTypes {
		types[i] = C.int32_t(t)
	}
	return call(func() C.int {
		return withChain(ch, func(cc *C.tcab_chain) C.int {
			return C.tcab_chain_prepare(cc, &types[0], C.uint32_t(len(types)), C.int(use), C.int(outDType))
		})
	})
}

// ReleaseStream frees the scratch memory the library allocated for launches
// on stream; call it before destroying a stream (tcab_release_stream).
func ReleaseStream(stream unsafe.Pointer) error {
	return call(func() C.int { return C.tcab_release_stream(stream) })
}

// Pipeline is tcab_pipeline: one operator over page-locked HOST buffers, cut
// into chunks of its independent axis (upload | kernel | download overlapped).
type Pipeline struct{ h *C.tcab_pipeline }

// NewSoftmaxPipeline streams fp32 rows of `cols` columns through
// tcab_softmax_rows on `device`, chunkRows rows at a time.
func NewSoftmaxPipeline(device int, cols, chunkRows uint32) (*Pipeline, error) {
	var d C.tcab_pipeline_desc
	d.op = C.TCAB_OP_SOFTMAX_ROWS
	d.device = C.int32_t(device)
	d.chunk_units = C.uint32_t(chunkRows)
	d.in_dtype = C.TCAB_F32
	d.n_streamed = 1
	d.unit_rank = 1
	d.unit_dims[0] = C.uint32_t(cols)
	p := &Pipeline{}
	if err := call(func() C.int { return C.tcab_pipeline_create(&d, &p.h) }); err != nil {
		return nil, err
	}
	return p, nil
}

// Run queues `units` units of the host buffers; Sync waits for them.
func (p *Pipeline) Run(hostIns []unsafe.Pointer, units uint64, hostOuts []unsafe.Pointer) error {
	return call(func() C.int {
		return C.tcab_pipeline_run(p.h, (*unsafe.Pointer)(unsafe.Pointer(&hostIns[0])), C.uint64_t(units),
			(*unsafe.Pointer)(unsafe.Pointer(&hostOuts[0])))
	})
}
func (p *Pipeline) Sync() error  { return call(func() C.int { return C.tcab_pipeline_sync(p.h) }) }
func (p *Pipeline) Close() error { return call(func() C.int { return C.tcab_pipeline_destroy(p.h) }) }

// HostAlloc returns page-locked host memory usable from every device.
func HostAlloc(bytes uint64) (unsafe.Pointer, error) {
	var p unsafe.Pointer
	err := call(func() C.int { return C.tcab_host_alloc(C.uint64_t(bytes), &p) })
	return p, err
}
