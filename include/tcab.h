/*
 * tcab.h -- C ABI of the B200 (sm_100a) map / reduce / contraction kernel library.
 *
 * This is the boundary a host written in another language (Go through cgo, C++,
 * Python through ctypes) binds. It replaces, for the operator classes below, the
 * launch layer the reference generates and links per kernel:
 *
 *   void <Name>Launch(const tca::Tensor<T,R>& in..., tca::Tensor<T,R>& out,
 *                     <scalar> s..., cudaStream_t stream);
 *       -- internal/cg/cxx/launch.go:23-156 (example: internal/cg/cxx/testdata/reduce_warp.cu:66-73)
 *
 * Conventions, mirroring that launcher:
 *   - tensors are NON-OWNING views of row-major contiguous device memory
 *     (runtime/tca/tensor.h:16-40); extents are 32-bit, element counts must stay
 *     below 2^32 (the reference indexes with u32);
 *   - every call is asynchronous on the CUDA stream passed in (NULL = the default
 *     stream) and runs on the CURRENT device; the caller synchronises;
 *   - shape agreement is checked before any launch, like the launcher's named
 *     TCA_REQUIREs (internal/cg/cxx/launch.go:23-156, runtime/tca/check.h:18-44);
 *   - where the reference throws std::runtime_error, these functions return a
 *     status code and leave a message for tcab_last_error() (a foreign caller
 *     cannot catch a C++ exception);
 *   - no entry point allocates device memory, except where its comment says so.
 *
 * There is no CPU fallback: without a CUDA device every compute entry point
 * returns TCAB_ERR_CUDA.
 */
#ifndef TCAB_H_
#define TCAB_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define TCAB_API __attribute__((visibility("default")))
#else
#define TCAB_API
#endif

#define TCAB_ABI_VERSION 1
#define TCAB_MAX_RANK 4
#define TCAB_MAX_INPUTS 6
#define TCAB_MAX_CAPTURES 8
#define TCAB_MAX_BATCH 32 /* problems tcab_chain_reduce_batched takes per call */
#define TCAB_PIPELINE_MAX_OUTPUTS 3
#define TCAB_NOALLOC_MAX_ROWS 4096 /* rows tcab_chain_reduce_noalloc accepts (its fixed scratch array) */

/* Status codes. 0 is success; everything else leaves a message for tcab_last_error(). */
typedef enum tcab_status {
  TCAB_OK = 0,
  TCAB_ERR_INVALID_ARG = 1, /* null pointer, bad enum value, rank out of range            */
  TCAB_ERR_SHAPE = 2,       /* operand shapes disagree (the launcher's TCA_REQUIRE class)  */
  TCAB_ERR_DTYPE = 3,       /* element type not supported by this operator class           */
  TCAB_ERR_ALIGNMENT = 4,   /* a pointer or extent breaks an alignment the kernel needs    */
  TCAB_ERR_UNSUPPORTED = 5, /* a lambda or size this build has no kernel for               */
  TCAB_ERR_CUDA = 6,        /* a CUDA runtime call or the launch itself failed             */
  TCAB_ERR_TOO_LARGE = 7    /* an extent beyond what the entry point states it accepts     */
} tcab_status;

/* Element types: the subset of internal/ir/types.go:13-24 these kernels move. */
typedef enum tcab_dtype {
  TCAB_F32 = 0,
  TCAB_BF16 = 1,
  TCAB_I32 = 2,
  TCAB_U32 = 3
} tcab_dtype;

/* Non-owning tensor view: the C spelling of tca::Tensor<T,R> (runtime/tca/tensor.h:16-40).
 * `data` is a device pointer; dims[0..rank) are the extents, slowest first. */
typedef struct tcab_tensor {
  void* data;
  int32_t dtype; /* tcab_dtype */
  uint32_t rank; /* 1..TCAB_MAX_RANK */
  uint32_t dims[TCAB_MAX_RANK];
} tcab_tensor;

/* A map | reduce | map chain, as the builder's rungs describe it
 * (pkg/chain.go:360-559: Iter -> Map -> As -> Reduce -> [Map -> As] -> Store).
 * Lambdas travel as C expressions in the reference's own operator and builtin vocabulary
 * (internal/cg/cxx/naming.go:126-198), typed the way the reference's builder types them
 * (pkg/expr.go:137-176, 185-203, 271):
 *   map_expr      over p0..p{n-1}, the operand values at the current point, each with its tensor's element
 *                 type, and c0..c{m-1}, the f32 scalar captures;   e.g. "(p0 * p1)"
 *   combine_expr  over p0 = accumulator, p1 = mapped value;        "(p0 + p1)", "fmaxf(p0, p1)", "fminf(p0, p1)"
 *   post_expr     piped map over p0 = the reduced value and c*; NULL when the chain stores the reduction as it is
 * Vocabulary: + - * / and unary - + on one arithmetic type (f32, i32, u32); % & | ^ << >> ~ on one integer
 * type; == != < <= > >= on one type, giving bool; && || ! on bool; cond ? a : b with two branches of one type;
 * static_cast<T>(x) with T one of float, __nv_bfloat16, int32_t, uint32_t (also spelled f32(x), bf16(x), i32(x),
 * u32(x)) between arithmetic types -- conversions are never implicit (internal/ir/types.go:60-62); the f32
 * builtins expf logf sqrtf rsqrtf fabsf tanhf sinf cosf fminf fmaxf fmaf and the u32 pair umin umax
 * (internal/ir/builtins.go:25-39). Literals: 1.5f / 1.5 / 2e-3 are f32, 3 is i32, 3u is u32, true / false bool.
 * bf16 is a storage type (design/syntax-design.md:601-607): a bf16 operand is converted before any arithmetic.
 * Converting a floating value that the integer type cannot hold is undefined, as in C++.
 * `init` is the reduction's initial value (an empty reduction returns it, design/tca.md:299). Reductions fold
 * f32 values: the map lambda of a reduce or contract chain must yield f32. */
typedef struct tcab_chain {
  const char* map_expr;
  const char* combine_expr;
  const char* post_expr;
  float init;
  uint32_t n_captures;
  float captures[TCAB_MAX_CAPTURES];
} tcab_chain;

/* Epilogue of the contraction (the piped map after the K reduction). */
typedef enum tcab_act {
  TCAB_ACT_NONE = 0,
  TCAB_ACT_RELU = 1 /* fmaxf(v, 0) */
} tcab_act;

/* Message of the calling thread's last failed call ("" if none). Replaces the text of the
 * std::runtime_error the reference throws (runtime/tca/check.h:18-44). */
TCAB_API const char* tcab_last_error(void);
TCAB_API const char* tcab_status_string(int status);
TCAB_API int tcab_abi_version(void);

/* Number of kernels this library has launched in the calling process (all threads). */
TCAB_API uint64_t tcab_launch_count(void);

/* Fused map + reduce over ONE axis of identically shaped operands, with an optional piped map:
 *   out[...] = post( fold_{k along reduce_axis} map(ins[0][..k..], ins[1][..k..], ...) )
 * Replaces the emitted reduce kernels and their launchers: one-tier sequential
 * (internal/cg/cxx/testdata/reduce_warp.cu:12-73), split-K warp reduce
 * (testdata/reduce_splitk.cu:13-91), amortised brackets (testdata/bracket_amort.cu:7-90),
 * i.e. SeqReducer / WarpReducer brackets (runtime/tca/reducer.h:36-181).
 * All operands: same rank (1..4) and extents, each f32, bf16, i32 or u32 (the map lambda sees each with its
 * own type and must yield f32). `out` is fp32 with the operands' extents minus the reduced axis (a rank-1
 * operand gives a rank-1 output of extent 1).
 * Operands that bind a subset of the iteration axes (the reference's structural indexing admits x[i] inside an
 * (i, j) iteration, pkg/chain.go checkOperand -- this is how a later statement reads a Local such as a row
 * maximum, pkg/local_test.go:17-68): when the reduced axis is the innermost one, an operand may have extent 1
 * along the innermost axis (one value per row) or extent 1 along every other axis (one row shared by all
 * rows: a bias, gamma, beta); when another axis is reduced, an operand may have extent 1 along the REDUCED axis
 * (one value per output cell: the column maxima of a middle-axis softmax). Such chains are compiled at run time;
 * rows with such operands are never split over CTAs.
 * reduce_axis == rank-1 selects the innermost-axis kernel, any other axis the outer-axis kernel.
 * The fold order is unspecified (design/tca.md:80-81,92); combine must be associative and commutative.
 * Allocation: when there are fewer rows than SMs and the rows are long, a row is split over several
 * CTAs (the multi-CTA reduction the reference stubs as GlobalReducer, runtime/tca/reducer.h:187-213) and
 * the partial results pass through 1 MiB of scratch memory that the library allocates with cudaMalloc
 * the first time a (device, stream) pair needs it and keeps until tcab_release_stream, tcab_release_all
 * or process exit. Make that first call outside any stream capture. A chain whose lambdas have no
 * ahead-of-time kernel is compiled on its first call (see tcab_chain_prepare). */
TCAB_API int tcab_chain_reduce(const tcab_chain* chain, const tcab_tensor* ins, uint32_t n_ins,
                      uint32_t reduce_axis, const tcab_tensor* out, void* stream);

/* tcab_chain_reduce over the INNERMOST axis for n_problems independent problems of ONE shape in one launch:
 *   outs[b][...] = post( fold_k map(ins[b * n_ins + 0][..k], ins[b * n_ins + 1][..k], ...) ),  b = 0..n_problems-1.
 * A lone small reduction is bounded by what a launch costs and by the wait for its predecessor on the stream,
 * not by memory: a [4096, 1024] fp32 input is 2.6 us of HBM time on a B200, and a dependent launch adds more
 * than a microsecond to it. A host that has several such problems (the rows of several layers, several
 * requests) hands them over together; the rows of all problems are one pool of work for the grid. The
 * reference's generated launcher takes one problem per call (internal/cg/cxx/launch.go:23-156).
 * ins: n_problems * n_ins tensors, problem-major, all of the shape and (per operand position) element type of
 * the first problem's; outs: n_problems f32 tensors with the operands' extents minus the innermost axis;
 * n_problems <= TCAB_MAX_BATCH. Pointers travel as kernel arguments: nothing is allocated, and rows are not
 * split over CTAs (long rows of few problems belong to tcab_chain_reduce). */
TCAB_API int tcab_chain_reduce_batched(const tcab_chain* chain, const tcab_tensor* ins, uint32_t n_ins,
                                       uint32_t n_problems, const tcab_tensor* outs, void* stream);

/* tcab_chain_reduce over the INNERMOST axis for callers that must not trigger a device allocation.
 * It has no counterpart in the reference. Who needs it: a host whose device memory is
 * already handed out in full (an embedding framework with its own arena, a serving process whose
 * pool was sized at start-up), code that runs while a CUDA graph is being captured, or a real-time
 * loop in which cudaMalloc's implicit device synchronisation is not acceptable. tcab_chain_reduce may
 * allocate 1 MiB per (device, stream) for the partial results of its multi-CTA split; this variant
 * runs the same split kernels with the partials in a fixed 16 KiB array that is part of the library's
 * device image (every GPU that loads the library holds it until the process exits), and calls neither
 * cudaMalloc nor cudaFree nor any allocating library routine -- nor the run-time compiler:
 *   - lambdas: the chain must have an ahead-of-time kernel or must already have been compiled in this
 *     process (by tcab_chain_prepare or by an earlier tcab_chain_reduce with the same lambdas). Compiling
 *     loads a code image onto the device, which is a device allocation, so this entry point never
 *     compiles: an unknown lambda is rejected with TCAB_ERR_UNSUPPORTED and a message that says so.
 *   - operands: fp32, identical shape; the reduced axis is the innermost one; the rows (the product of
 *     the other extents) may number at most TCAB_NOALLOC_MAX_ROWS, because every row needs at least one
 *     slot of the array. More rows are rejected with TCAB_ERR_TOO_LARGE; use tcab_chain_reduce then.
 *   - the first call on a device looks up the array's device address (cudaGetSymbolAddress, with that
 *     device current). Make that first call before any stream capture begins.
 *   - all calls on a device share the one array. It keeps the previous call's partial results; nothing
 *     in it needs clearing, because a call writes every slot it later reads. Two calls that overlap on
 *     the GPU (different streams, or different host threads on different streams) race on it: order
 *     them on one stream or with events. */
TCAB_API int tcab_chain_reduce_noalloc(const tcab_chain* chain, const tcab_tensor* ins, uint32_t n_ins,
                                       const tcab_tensor* out, void* stream);

/* Compiles and loads, now, the kernels that the first tcab_chain_reduce (use = TCAB_USE_REDUCE),
 * tcab_chain_contract (use = TCAB_USE_CONTRACT, n_ins = 2), tcab_map (use = TCAB_USE_MAP) or
 * tcab_chain_reduce_batched (use = TCAB_USE_REDUCE_BATCHED) with these lambdas
 * and operand element types (in_dtypes: n_ins tcab_dtype values, NULL = all f32; out_dtype: the stored type of
 * a map, ignored otherwise) would otherwise compile on its first call. The reference compiles every kernel ahead of time from its lambdas
 * (internal/cg/cxx/emit.go:85-190 prints the translation unit, the user runs nvcc); this is the same step
 * for a lambda that this library has no ahead-of-time kernel for. It takes hundreds of milliseconds, loads a
 * code image onto the current device (an implicit device allocation) and must not run during a stream
 * capture. Lambdas that have an ahead-of-time kernel return at once. Only the lambdas and the operand count
 * matter; `init` and the capture values may differ in later calls. */
#define TCAB_USE_REDUCE 0
#define TCAB_USE_CONTRACT 1
#define TCAB_USE_MAP 2
#define TCAB_USE_REDUCE_BATCHED 3
TCAB_API int tcab_chain_prepare(const tcab_chain* chain, const int32_t* in_dtypes, uint32_t n_ins, int use,
                                int out_dtype);

/* Map-only chain with a rank-preserving store: out[i...] = map_expr(ins[0][i...], ins[1][i...], ...).
 * The fused elementwise map of the path. The reference's rungs cannot store a map that no reduction
 * follows (pkg/chain.go:433-438 admits Store only after a Reduce), so, like the softmax and layer-norm
 * chains, it is offered as an entry point of its own; what it replaces in the emitted code is the per-element
 * TensorView::Get / Set pair (runtime/tca/view.h:104-112) of a map statement.
 * ins: 1..TCAB_MAX_INPUTS tensors of the shape of `out`, each f32, bf16, i32 or u32; the lambda sees every
 * operand with its own element type and must yield exactly the element type of `out` (no implicit conversion).
 * An operand may also have the rank of `out` with extent 1 along the innermost axis (one value per row: the
 * row maximum of a softmax) or extent 1 along every other axis (one row shared by all rows: a bias), the two
 * subsets of the iteration axes an operand of the reference may bind (pkg/chain.go checkOperand).
 * Only chain->map_expr, n_captures and captures are read. Every element is computed once, in IEEE fp32
 * arithmetic per operation with CUDA's math functions (expf ... fmaf: at most 2 ulp from the exact value). */
TCAB_API int tcab_map(const tcab_chain* chain, const tcab_tensor* ins, uint32_t n_ins, const tcab_tensor* out,
                      void* stream);

/* Contraction chain over operands indexed by different dim subsets:
 *   out[m,n] = post( fold_k map(lhs[m,k], rhs[k,n]) )   rhs_is_nk == 0, rhs is [K,N]
 *   out[m,n] = post( fold_k map(lhs[m,k], rhs[n,k]) )   rhs_is_nk != 0, rhs is [N,K]
 * with the lambdas of tcab_chain (map over p0 = the lhs value, p1 = the rhs value). Replaces the emitted
 * matmul-shaped kernels of the reference's suite (testing/kernels/llm/gemm.tca, llm/qk_score.tca,
 * tiling/mm_small.tca, mm_mid.tca, mm_splitk.tca, fusion/mlp.tca; launcher form
 * internal/cg/cxx/launch.go:23-156). Each output is folded over k in ascending order, the order of the
 * reference's CPU loops (testing/runners/gemm.cu:44-56). lhs and rhs are f32, bf16, i32 or u32 (a bf16
 * operand is widened at the load; the lambda converts it explicitly, e.g. "f32(p0) * f32(p1)", the spelling of
 * testing/kernels/llm/qk_score.tca with bf16 storage); out is f32. Any lambda runs in fp32 arithmetic on the
 * scalar pipes. One chain runs on the tensor cores instead (fp32 accumulation, fp32 store, the same launch
 * count): both operands bf16, map the plain product "f32(p0) * f32(p1)", a sum reducer with init 0, no piped map
 * or a scaling by one constant ("p0 * c0", "0.5f * p0"), K a multiple of 8, N a multiple of 4 (of 8 when rhs is
 * [K,N]) and 16-byte aligned pointers. Products of bf16 values are exact in fp32, so only the order in which an
 * output's k terms are added differs from the scalar kernel. The same chain over two f32 operands ("p0 * p1")
 * takes the tensor cores from m * n * k = 2^29 on (K >= 256, K a multiple of 4): each operand is cut
 * into three bf16 pieces (24 significant bits) in a workspace of 12 bytes per operand element (per device and
 * stream, at most 512 MiB; larger problems run in blocks), and the six significant piece products are one bf16
 * contraction over 6 K; what is dropped is below 3 * 2^-24 of |a b| per product (measured: 3e-7 .. 8e-7 of
 * sum |a||b| per output, the same as an fp32 library GEMM). Smaller problems keep the scalar kernel and with it
 * the reference's ascending order over k. */
TCAB_API int tcab_chain_contract(const tcab_chain* chain, const tcab_tensor* lhs, const tcab_tensor* rhs,
                                 int rhs_is_nk, const tcab_tensor* out, void* stream);

/* Outer-axis reduce of t[b, k, c] over k in ONE pass: any of sum (fp32), max (fp32) and argmax
 * (int32, lowest index among equal maxima) may be NULL. Each output is [b, c].
 * The reference's class: the middle-axis kernels of testing/kernels/runtime/row_sum.tca:18-33 and
 * testing/kernels/fusion/softmax.tca; argmax has no spelling in the reference's reducers
 * (pkg/chain.go:242-260 admits homogeneous scalar reducers only), so it is offered here directly. */
TCAB_API int tcab_reduce_outer(const tcab_tensor* t, const tcab_tensor* sum, const tcab_tensor* max,
                      const tcab_tensor* argmax, void* stream);

/* Row softmax, y[i,j] = expf(x[i,j]-m_i) / sum_j expf(x[i,j]-m_i), m_i = max_j x[i,j]:
 * the map | reduce | map chain over the innermost axis with a rank-preserving store. The reference's
 * rungs cannot store a rank-preserving map (pkg/chain.go:433-438; the shipped
 * testing/kernels/fusion/softmax.tca is its fallback), so the chain is one entry point.
 * x, y: fp32, same shape, rank 1..4; rows are the innermost axis. */
TCAB_API int tcab_softmax_rows(const tcab_tensor* x, const tcab_tensor* y, void* stream);

/* Layer-norm over the innermost axis with fp32 statistics:
 *   y = (x - mean) / sqrtf(var + eps) * gamma + beta,  mean = sum(x)/n,  var = sum((x-mean)^2)/n.
 * x, y: bf16 or fp32 (same type and shape); gamma, beta: rank 1, extent = the innermost extent,
 * same element type as x. The reference's fallback for this chain is
 * testing/kernels/llm/layernorm.tca:1-40 (runner testing/runners/layernorm.cu:47-58). */
TCAB_API int tcab_layernorm_rows(const tcab_tensor* x, const tcab_tensor* gamma, const tcab_tensor* beta,
                        float eps, const tcab_tensor* y, void* stream);

/* Tiled contraction with a fused epilogue: c = act(a @ b + bias).
 * a [M,K] bf16, b [K,N] bf16, bias [N] fp32 or NULL, c [M,N] bf16; fp32 accumulation.
 * Replaces the emitted GEMM (one output element per CTA bracket; the suite's
 * testing/kernels/llm/gemm.tca, runner testing/runners/gemm.cu:44-56) plus the piped map the
 * reference's final-lower cannot bind a tensor operand to (design/RELEASE-v0.0.0.md:150).
 * Requires K % 8 == 0, N % 8 == 0 and 16-byte aligned base pointers (TMA tensor maps). */
TCAB_API int tcab_gemm_bias_act(const tcab_tensor* a, const tcab_tensor* b, const tcab_tensor* bias,
                       int act, const tcab_tensor* c, void* stream);

/* ---------------------------------------------------------------------------------------------------
 * Host buffers: upload, kernel and download pipelined over chunks of the independent axis.
 *
 * The entry points above take device tensors and leave the copies to the caller, like the reference's
 * launchers; the reference's own runners copy whole tensors around the launch
 * (testing/runners/common.cuh:72-90: cudaMemcpy in, launch, synchronise, cudaMemcpy out), which serialises the
 * two PCIe directions around the kernel. Every operator class here has an axis along which outputs are
 * independent -- rows (softmax, layer-norm, chain_reduce over the innermost axis, map), the batch of
 * reduce_outer, the rows of a in the contraction -- so a problem in host memory is cut into chunks of that
 * axis: chunk i+1 uploads while chunk i computes and chunk i-1 downloads, on three streams that the pipeline
 * owns. A "unit" is one index of the independent axis; the streamed operands hold `units` of them.
 *
 * A pipeline owns: three non-blocking streams, `depth` staging slots in device memory (each chunk_units units
 * of every streamed operand and every output), three events per slot. tcab_pipeline_create allocates them
 * (cudaMalloc), tcab_pipeline_destroy frees them after waiting for the pipeline's work. Host buffers should be
 * page-locked (tcab_host_alloc, cudaHostAlloc / cudaHostRegister, or torch's pin_memory): with pageable memory
 * the copies are staged by the driver and do not overlap. A pipeline may be used from one host thread at a
 * time. There is no CPU fallback: without a device tcab_pipeline_create returns TCAB_ERR_CUDA.
 * --------------------------------------------------------------------------------------------------- */
typedef enum tcab_op {
  TCAB_OP_SOFTMAX_ROWS = 0,   /* unit: a row [cols] f32                -> y row, resident: none             */
  TCAB_OP_LAYERNORM_ROWS = 1, /* unit: a row [cols] f32 / bf16         -> y row, resident: gamma, beta; eps */
  TCAB_OP_REDUCE_OUTER = 2,   /* unit: one batch [k, c] f32            -> sum, max, argmax [c] (by `outputs`) */
  TCAB_OP_CHAIN_REDUCE = 3,   /* unit: a row [cols] f32 / bf16 of each of n_streamed operands -> one f32; chain */
  TCAB_OP_GEMM_BIAS_ACT = 4,  /* unit: a row of a [K] bf16             -> row of c [N] bf16, resident: b [K,N], bias [N] or none; act */
  TCAB_OP_MAP = 5             /* unit: any shape, n_streamed operands of in_dtype -> same shape, out_dtype; chain */
} tcab_op;

typedef struct tcab_pipeline_desc {
  int32_t op;            /* tcab_op */
  int32_t device;        /* CUDA ordinal the pipeline runs on; -1 = the device current at create */
  uint32_t chunk_units;  /* units per chunk (the last chunk of a run may be shorter) */
  uint32_t depth;        /* staging slots, 2..8; 0 = 4 */
  int32_t in_dtype;      /* tcab_dtype of the streamed operand(s) */
  uint32_t n_streamed;   /* streamed operands: 1, or 1..TCAB_MAX_INPUTS for CHAIN_REDUCE and MAP */
  uint32_t unit_rank;    /* rank of one unit, 1..TCAB_MAX_RANK-1 */
  uint32_t unit_dims[TCAB_MAX_RANK - 1];
  uint32_t outputs;      /* REDUCE_OUTER: bit 0 sum, bit 1 max, bit 2 argmax; host_outs lists the chosen ones in that order */
  int32_t out_dtype;     /* MAP: tcab_dtype of the result */
  int32_t act;           /* GEMM_BIAS_ACT: tcab_act */
  float eps;             /* LAYERNORM_ROWS */
  const tcab_chain* chain; /* CHAIN_REDUCE, MAP: the lambdas (copied at create) */
  tcab_tensor resident[2]; /* operands that stay in device memory (on `device`): gamma, beta | b, bias (data NULL = none) */
} tcab_pipeline_desc;

typedef struct tcab_pipeline tcab_pipeline;

TCAB_API int tcab_pipeline_create(const tcab_pipeline_desc* desc, tcab_pipeline** out);
/* Number of host output buffers a run takes (1, or the number of bits set in `outputs`). */
TCAB_API uint32_t tcab_pipeline_outputs(const tcab_pipeline* p);
/* Queues `units` units: host_ins[i] holds units * (unit elements) of streamed operand i, host_outs[j] receives the
 * j-th output. Returns once everything is queued (with page-locked buffers nothing waits on the host); runs may
 * follow each other without a join in between -- the first uploads of the next run then overlap the last
 * downloads of this one. The buffers must stay valid until tcab_pipeline_sync or a stream joined after the run
 * has passed. */
TCAB_API int tcab_pipeline_run(tcab_pipeline* p, const void* const* host_ins, uint64_t units, void* const* host_outs);
/* Work queued on the pipeline after this call starts only once everything queued on `stream` so far is done. */
TCAB_API int tcab_pipeline_order_after(tcab_pipeline* p, void* stream);
/* `stream` waits (on the device, not the host) for everything queued on the pipeline so far. */
TCAB_API int tcab_pipeline_join(tcab_pipeline* p, void* stream);
/* The calling host thread waits for everything queued on the pipeline so far. */
TCAB_API int tcab_pipeline_sync(tcab_pipeline* p);
TCAB_API int tcab_pipeline_destroy(tcab_pipeline* p);

/* One problem in host memory cut over several devices of this process: device r of n takes the contiguous
 * block tcab_shard_block(units, n, r) of the independent axis through a pipeline of its own (descs[r], whose
 * `device` fields must name distinct devices and whose resident operands live on that device: gamma / beta or
 * b / bias are replicated by the caller beforehand). No device exchanges anything with another: the path has no
 * data-path collective. The reference has no multi-device support (internal/cg/cxx/loops.go:11-22 spreads loop
 * dims over CTAs and warps of one GPU only). Chunks are queued round-robin over the devices. */
typedef struct tcab_multi tcab_multi;
TCAB_API int tcab_multi_create(const tcab_pipeline_desc* descs, uint32_t n_devices, tcab_multi** out);
TCAB_API int tcab_multi_run(tcab_multi* m, const void* const* host_ins, uint64_t units, void* const* host_outs);
TCAB_API int tcab_multi_sync(tcab_multi* m);
TCAB_API int tcab_multi_destroy(tcab_multi* m);

/* The partition rule: [*lo, *hi) is the contiguous block rank `rank` of `world` owns out of n units. Blocks
 * differ by at most one unit, the first n % world ranks get the larger ones, every unit belongs to one rank. */
TCAB_API int tcab_shard_block(uint64_t n, uint32_t world, uint32_t rank, uint64_t* lo, uint64_t* hi);

/* Page-locked host memory usable from every device (cudaHostAlloc with the portable flag), for hosts that
 * cannot call the CUDA runtime themselves (a cgo host). */
TCAB_API int tcab_host_alloc(uint64_t bytes, void** out);
TCAB_API int tcab_host_free(void* p);

/* Scratch memory the library allocated for launches on `stream` of the current device (the multi-CTA
 * partials of tcab_chain_reduce: 1 MiB; of tcab_reduce_outer: 3 MiB; the K-range workspace of
 * tcab_gemm_bias_act: up to 64 MiB) is freed; tcab_release_all frees it for every device and stream. A host
 * that creates and destroys streams calls tcab_release_stream before destroying one. cudaFree waits for the
 * device to go idle, so neither call may run during a stream capture. No counterpart in the reference, whose
 * launchers own no memory (internal/cg/cxx/launch.go:23-156). */
TCAB_API int tcab_release_stream(void* stream);
TCAB_API int tcab_release_all(void);

/* Reads the device-side status word of the current device into *status (a synchronous copy):
 * 0 = no kernel of this library has given up on a bounded wait since the library was loaded,
 * non-zero = a contraction kernel abandoned a barrier wait and returned early (its output is then
 * incomplete). The reference's device-side failure path is a device assert (runtime/tca/reducer.h:198-206);
 * this library never traps: it reports here. */
TCAB_API int tcab_device_status(int* status);

#ifdef __cplusplus
}
#endif

#endif /* TCAB_H_ */
