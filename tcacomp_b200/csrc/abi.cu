// abi.cu -- the extern "C" surface declared in include/tcab.h: argument and shape
// validation, then one launch into the operator-class kernels.
//
// The checks stand where the reference's generated launcher derives every
// extent from its first tensor occurrence and TCA_REQUIREs the others to agree
// (internal/cg/cxx/launch.go:23-156), and where ValidateLaunch traps bad launch
// geometry (runtime/tca/launch.h:37-58). A failure is a status code plus a
// thread-local message; nothing throws across the boundary.
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <map>
#include <mutex>
#include <utility>

#include "../../include/tcab_tuning.h"
#include "common.cuh"
#include "rowvec.cuh"

namespace tcab {
namespace {

thread_local char g_err[512] = "";
std::atomic<uint64_t> g_launches{0};
Tune g_tune[kFamilies];

struct DevFacts {
  int sms = 0;
  int optin_smem = 0;
};
std::mutex g_mu;
std::map<int, DevFacts> g_dev;
std::map<std::pair<std::pair<int, const void*>, std::pair<int, size_t>>, int> g_occ;

int current_device() {
  int d = 0;
  if (cudaGetDevice(&d) != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  return d;
}

const DevFacts& facts() {
  static const DevFacts none{};
  const int d = current_device();
  if (d < 0) return none;
  std::lock_guard<std::mutex> lk(g_mu);
  auto it = g_dev.find(d);
  if (it == g_dev.end()) {
    DevFacts f;
    cudaDeviceGetAttribute(&f.sms, cudaDevAttrMultiProcessorCount, d);
    cudaDeviceGetAttribute(&f.optin_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, d);
    it = g_dev.emplace(d, f).first;
  }
  return it->second;
}

}  // namespace

int fail(int status, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  std::vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return status;
}

void count_launch(unsigned n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

int sm_count() {
  const int n = facts().sms;
  return n > 0 ? n : 1;
}

int max_optin_smem() { return facts().optin_smem; }

int check_launch(const char* what) {
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(TCAB_ERR_CUDA, "%s: launch failed: %s", what, cudaGetErrorString(e));
  return TCAB_OK;
}

const Tune& tune(int family) { return g_tune[family]; }

int occupancy(const void* fn, int block, size_t smem) {
  const int d = current_device();
  const auto key = std::make_pair(std::make_pair(d, fn), std::make_pair(block, smem));
  {
    std::lock_guard<std::mutex> lk(g_mu);
    auto it = g_occ.find(key);
    if (it != g_occ.end()) return it->second;
  }
  int n = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, fn, block, smem) != cudaSuccess) {
    cudaGetLastError();
    n = 1;
  }
  std::lock_guard<std::mutex> lk(g_mu);
  g_occ[key] = n;
  return n;
}

namespace {
struct ScratchBuf {
  void* p = nullptr;
  size_t bytes = 0;
};
std::mutex g_scratch_mu;
std::map<std::pair<std::pair<int, cudaStream_t>, int>, ScratchBuf> g_scratch;
}  // namespace

void* stream_scratch(int kind, cudaStream_t stream, size_t bytes, bool grow, bool zero) {
  const int dev = current_device();
  if (dev < 0) return nullptr;
  std::lock_guard<std::mutex> lk(g_scratch_mu);
  ScratchBuf& b = g_scratch[{{dev, stream}, kind}];
  if (b.p != nullptr && b.bytes >= bytes) return b.p;
  if (b.p != nullptr) {
    if (!grow) return nullptr;
    cudaFree(b.p);
    b = ScratchBuf{};
  }
  if (cudaMalloc(&b.p, bytes) != cudaSuccess || (zero && cudaMemset(b.p, 0, bytes) != cudaSuccess)) {
    cudaGetLastError();
    if (b.p != nullptr) cudaFree(b.p);
    b = ScratchBuf{};
    return nullptr;
  }
  b.bytes = bytes;
  return b.p;
}

namespace {

// Frees the buffers of one (device, stream), or all of them. cudaFree waits for the device to go idle.
void release_scratch(bool all, int dev, cudaStream_t stream) {
  std::lock_guard<std::mutex> lk(g_scratch_mu);
  for (auto it = g_scratch.begin(); it != g_scratch.end();) {
    if (all || (it->first.first.first == dev && it->first.first.second == stream)) {
      if (it->second.p != nullptr) cudaFree(it->second.p);
      it = g_scratch.erase(it);
    } else {
      ++it;
    }
  }
  cudaGetLastError();
}

// ---- validation helpers ----------------------------------------------------

int check_tensor(const char* op, const char* name, const tcab_tensor* t, bool need_data = true) {
  if (t == nullptr) return fail(TCAB_ERR_INVALID_ARG, "%s: tensor '%s' is null", op, name);
  if (t->rank < 1 || t->rank > TCAB_MAX_RANK)
    return fail(TCAB_ERR_INVALID_ARG, "%s: tensor '%s' has rank %u (want 1..%d)", op, name, t->rank, TCAB_MAX_RANK);
  uint64_t n = 1;
  for (uint32_t i = 0; i < t->rank; ++i) {
    n *= t->dims[i];
    if (n >= (1ull << 32))
      return fail(TCAB_ERR_TOO_LARGE, "%s: tensor '%s' has 2^32 or more elements", op, name);
  }
  if (need_data && n > 0 && t->data == nullptr)
    return fail(TCAB_ERR_INVALID_ARG, "%s: tensor '%s' has a null data pointer", op, name);
  return TCAB_OK;
}

uint64_t count(const tcab_tensor* t, uint32_t from, uint32_t to) {
  uint64_t n = 1;
  for (uint32_t i = from; i < to; ++i) n *= t->dims[i];
  return n;
}

bool same_shape(const tcab_tensor* a, const tcab_tensor* b) {
  if (a->rank != b->rank) return false;
  for (uint32_t i = 0; i < a->rank; ++i)
    if (a->dims[i] != b->dims[i]) return false;
  return true;
}

int need_dtype(const char* op, const char* name, const tcab_tensor* t, int dtype, const char* spelled) {
  if (t->dtype != dtype) return fail(TCAB_ERR_DTYPE, "%s: tensor '%s' must be %s", op, name, spelled);
  return TCAB_OK;
}

int need_elem_align(const char* op, const char* name, const tcab_tensor* t, unsigned bytes) {
  if (reinterpret_cast<uintptr_t>(t->data) % bytes != 0)
    return fail(TCAB_ERR_ALIGNMENT, "%s: tensor '%s' is not %u-byte aligned", op, name, bytes);
  return TCAB_OK;
}

// Element types a lambda operand may have (the chain and map classes): 4-byte f32 / i32 / u32, 2-byte bf16.
int need_operand_dtype(const char* op, const char* name, const tcab_tensor* t) {
  if (t->dtype != TCAB_F32 && t->dtype != TCAB_BF16 && t->dtype != TCAB_I32 && t->dtype != TCAB_U32)
    return fail(TCAB_ERR_DTYPE, "%s: tensor '%s' must be f32, bf16, i32 or u32", op, name);
  return need_elem_align(op, name, t, t->dtype == TCAB_BF16 ? 2 : 4);
}

// How an operand of the iteration shape `full` (rank r) is indexed: 0 = by every axis (same shape), 1 = one value
// per row (full's extents with the innermost one = 1), 2 = one row shared by all rows (every extent 1 but the
// innermost), -1 = none of these. The reference lets an operand bind a subset of the live axes
// (pkg/chain.go checkOperand); these are the two subsets the innermost-axis kernels take.
int operand_indexing(const uint32_t* full, uint32_t rank, const tcab_tensor* t) {
  if (t->rank != rank) return -1;
  bool same = true, row = t->dims[rank - 1] == 1, col = t->dims[rank - 1] == full[rank - 1];
  for (uint32_t i = 0; i < rank; ++i) same = same && t->dims[i] == full[i];
  for (uint32_t i = 0; i + 1 < rank; ++i) {
    row = row && t->dims[i] == full[i];
    col = col && t->dims[i] == 1;
  }
  if (same) return 0;
  if (row) return 1;
  if (col && rank > 1) return 2;
  return -1;
}

int have_device(const char* op) {
  if (current_device() < 0) return fail(TCAB_ERR_CUDA, "%s: no CUDA device (this library has no CPU path)", op);
  return TCAB_OK;
}

#define TCAB_TRY(expr)              \
  do {                              \
    const int tcab_rc_ = (expr);    \
    if (tcab_rc_ != TCAB_OK) return tcab_rc_; \
  } while (0)

}  // namespace
}  // namespace tcab

using namespace tcab;

extern "C" {

const char* tcab_last_error(void) { return g_err; }

const char* tcab_status_string(int status) {
  switch (status) {
    case TCAB_OK: return "ok";
    case TCAB_ERR_INVALID_ARG: return "invalid argument";
    case TCAB_ERR_SHAPE: return "shape mismatch";
    case TCAB_ERR_DTYPE: return "unsupported element type";
    case TCAB_ERR_ALIGNMENT: return "misaligned operand";
    case TCAB_ERR_UNSUPPORTED: return "unsupported by this build";
    case TCAB_ERR_CUDA: return "CUDA failure";
    case TCAB_ERR_TOO_LARGE: return "extent too large";
    default: return "unknown status";
  }
}

int tcab_abi_version(void) { return TCAB_ABI_VERSION; }

uint64_t tcab_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int tcab_device_status(int* status) {
  if (status == nullptr) return fail(TCAB_ERR_INVALID_ARG, "device_status: null output");
  TCAB_TRY(have_device("device_status"));
  int gemm = 0, rows = 0;
  TCAB_TRY(gemm_device_status(&gemm));
  TCAB_TRY(rows_smem_status(&rows));
  *status = gemm != 0 ? gemm : (rows != 0 ? 16 : 0);  // 1..4: a contraction kernel, 16: a shared-memory row kernel
  return TCAB_OK;
}

int tcab_release_stream(void* stream) {
  TCAB_TRY(have_device("release_stream"));
  release_scratch(false, current_device(), static_cast<cudaStream_t>(stream));
  return TCAB_OK;
}

int tcab_release_all(void) {
  release_scratch(true, 0, nullptr);
  return TCAB_OK;
}

namespace {
int prepare_common(const char* op, const tcab_chain* chain, const int32_t* in_dtypes, uint32_t n_ins, int use, int out_dtype,
                   PreparedChain* pc);
}

int tcab_compile_check(const tcab_chain* chain, const int32_t* in_dtypes, uint32_t n_ins, int use, int out_dtype,
                       int row_value_mask, int shared_row_mask, int cell_value_mask) {
  PreparedChain pc;
  TCAB_TRY(prepare_common("compile_check", chain, in_dtypes, n_ins, use, out_dtype, &pc));
  JitSpec sp = pc.spec;
  sp.rb_mask = row_value_mask;
  sp.cb_mask = shared_row_mask;
  sp.cell_mask = cell_value_mask;
  return jit_compile_check(sp);
}

int tcab_chain_prepare(const tcab_chain* chain, const int32_t* in_dtypes, uint32_t n_ins, int use, int out_dtype) {
  const char* op = "chain_prepare";
  PreparedChain pc;
  TCAB_TRY(prepare_common(op, chain, in_dtypes, n_ins, use, out_dtype, &pc));
  TCAB_TRY(have_device(op));
  return warm_chain(pc);
}

namespace {
int prepare_common(const char* op, const tcab_chain* chain, const int32_t* in_dtypes, uint32_t n_ins, int use, int out_dtype,
                   PreparedChain* pcp) {
  PreparedChain& pc = *pcp;
  if (chain == nullptr || chain->map_expr == nullptr)
    return fail(TCAB_ERR_INVALID_ARG, "%s: chain and map_expr are required", op);
  if (use != TCAB_USE_REDUCE && use != TCAB_USE_CONTRACT && use != TCAB_USE_MAP && use != TCAB_USE_REDUCE_BATCHED)
    return fail(TCAB_ERR_INVALID_ARG, "%s: unknown use %d", op, use);
  if (use != TCAB_USE_MAP && chain->combine_expr == nullptr) return fail(TCAB_ERR_INVALID_ARG, "%s: combine_expr is required", op);
  if (chain->n_captures > TCAB_MAX_CAPTURES)
    return fail(TCAB_ERR_INVALID_ARG, "%s: %u captures (at most %d)", op, chain->n_captures, TCAB_MAX_CAPTURES);
  if (n_ins < 1 || n_ins > TCAB_MAX_INPUTS || (use == TCAB_USE_CONTRACT && n_ins != 2))
    return fail(TCAB_ERR_INVALID_ARG, "%s: bad operand count %u", op, n_ins);
  int types[TCAB_MAX_INPUTS] = {};  // TCAB_F32 == 0
  for (uint32_t i = 0; i < n_ins && in_dtypes != nullptr; ++i) {
    if (in_dtypes[i] < TCAB_F32 || in_dtypes[i] > TCAB_U32) return fail(TCAB_ERR_DTYPE, "%s: in_dtypes[%u] is not a tcab_dtype", op, i);
    types[i] = in_dtypes[i];
  }
  if (use == TCAB_USE_MAP && (out_dtype < TCAB_F32 || out_dtype > TCAB_U32)) return fail(TCAB_ERR_DTYPE, "%s: out_dtype is not a tcab_dtype", op);
  TCAB_TRY(prepare_chain(chain, n_ins, &pc, use == TCAB_USE_MAP ? 'M' : use == TCAB_USE_CONTRACT ? 'C' : 'R', types,
                         use == TCAB_USE_MAP ? out_dtype : TCAB_F32));
  if (use == TCAB_USE_REDUCE_BATCHED) pc.spec.kind = 'B';
  return TCAB_OK;
}
}  // namespace

int tcab_tune(const char* family, int p0, int p1, int p2, int p3) {
  static const char* names[kFamilies] = {"softmax", "layernorm", "reduce_inner", "reduce_outer", "gemm"};
  if (family == nullptr) return fail(TCAB_ERR_INVALID_ARG, "tune: null family");
  for (int i = 0; i < kFamilies; ++i) {
    if (std::strcmp(family, names[i]) == 0) {
      g_tune[i].p0 = p0 > 0 ? p0 : 0;
      g_tune[i].p1 = p1 > 0 ? p1 : 0;
      g_tune[i].p2 = p2 > 0 ? p2 : 0;
      g_tune[i].p3 = p3 > 0 ? p3 : 0;
      return TCAB_OK;
    }
  }
  return fail(TCAB_ERR_INVALID_ARG, "tune: unknown family '%s'", family);
}

int tcab_plan_outer_split(uint64_t tiles, uint64_t cells, uint32_t nk, uint64_t resident_ctas, int sms, int forced,
                          uint32_t* ranges, uint32_t* klen) {
  if (ranges == nullptr || klen == nullptr) return fail(TCAB_ERR_INVALID_ARG, "plan_outer_split: null output");
  if (sms < 1) return fail(TCAB_ERR_INVALID_ARG, "plan_outer_split: sms must be positive");
  plan_outer_ranges(plan_outer_splits(tiles, cells, nk, resident_ctas, sms, forced), nk, ranges, klen);
  return TCAB_OK;
}

int tcab_plan_row_kernels(uint64_t rows_or_batches, uint32_t nk, uint32_t nc, int sms, uint32_t nvec, uint32_t per_step,
                          int prefer_three, int n_in, uint32_t* outer_flat_g, uint32_t* stream_cluster, uint32_t* rows32) {
  if (outer_flat_g == nullptr || stream_cluster == nullptr || rows32 == nullptr)
    return fail(TCAB_ERR_INVALID_ARG, "plan_row_kernels: null output");
  if (sms < 1 || per_step < 1) return fail(TCAB_ERR_INVALID_ARG, "plan_row_kernels: sms and per_step must be positive");
  *outer_flat_g = outer_flat_groups(rows_or_batches, nk, nc, sms, nc % 4 == 0);
  *stream_cluster = stream_cluster_size(nvec, per_step, prefer_three != 0);
  *rows32 = rows32_warps(nvec, n_in);
  return TCAB_OK;
}

int tcab_plan_row_shape(int op, int elem_bytes, uint32_t nvec, uint32_t* threads_per_row, uint32_t* slots_per_thread) {
  if (threads_per_row == nullptr || slots_per_thread == nullptr) return fail(TCAB_ERR_INVALID_ARG, "plan_row_shape: null output");
  if ((op != 0 && op != 1) || (elem_bytes != 2 && elem_bytes != 4) || (op == 0 && elem_bytes != 4))
    return fail(TCAB_ERR_INVALID_ARG, "plan_row_shape: op 0 (softmax, 4-byte elements) or 1 (layer-norm, 2 or 4)");
  int t = 0, v = 0;
  const bool fits = op == 0 ? tcab::softmax_row_shape(nvec, true, &t, &v) : tcab::layernorm_row_shape(nvec, true, elem_bytes, &t, &v);
  *threads_per_row = fits ? static_cast<uint32_t>(t) : 0;
  *slots_per_thread = fits ? static_cast<uint32_t>(v) : 0;
  return TCAB_OK;
}

int tcab_plan_outer_flat_ranges(uint64_t batches, uint32_t nk, uint32_t nc, int sms, uint64_t max_partials,
                                uint32_t* groups, uint32_t* ranges, uint32_t* klen) {
  if (groups == nullptr || ranges == nullptr || klen == nullptr)
    return fail(TCAB_ERR_INVALID_ARG, "plan_outer_flat_ranges: null output");
  if (sms < 1) return fail(TCAB_ERR_INVALID_ARG, "plan_outer_flat_ranges: sms must be positive");
  *groups = outer_flat_groups(batches, nk, nc, sms, nc % 4 == 0);
  *ranges = 1;
  *klen = nk;
  if (*groups != 0) *ranges = outer_flat_ranges(batches, nk, nc, *groups, nc % 4 == 0, sms, max_partials, klen);
  return TCAB_OK;
}

int tcab_softmax_rows(const tcab_tensor* x, const tcab_tensor* y, void* stream) {
  const char* op = "softmax_rows";
  TCAB_TRY(check_tensor(op, "x", x));
  TCAB_TRY(check_tensor(op, "y", y));
  TCAB_TRY(need_dtype(op, "x", x, TCAB_F32, "f32"));
  TCAB_TRY(need_dtype(op, "y", y, TCAB_F32, "f32"));
  if (!same_shape(x, y)) return fail(TCAB_ERR_SHAPE, "%s: y must have the shape of x", op);
  TCAB_TRY(need_elem_align(op, "x", x, 4));
  TCAB_TRY(need_elem_align(op, "y", y, 4));
  TCAB_TRY(have_device(op));
  const uint32_t cols = x->dims[x->rank - 1];
  return launch_softmax_rows(static_cast<const float*>(x->data), static_cast<float*>(y->data),
                             count(x, 0, x->rank - 1), cols, static_cast<cudaStream_t>(stream));
}

int tcab_layernorm_rows(const tcab_tensor* x, const tcab_tensor* gamma, const tcab_tensor* beta, float eps,
                        const tcab_tensor* y, void* stream) {
  const char* op = "layernorm_rows";
  TCAB_TRY(check_tensor(op, "x", x));
  TCAB_TRY(check_tensor(op, "gamma", gamma));
  TCAB_TRY(check_tensor(op, "beta", beta));
  TCAB_TRY(check_tensor(op, "y", y));
  if (x->dtype != TCAB_F32 && x->dtype != TCAB_BF16) return fail(TCAB_ERR_DTYPE, "%s: x must be f32 or bf16", op);
  if (y->dtype != x->dtype || gamma->dtype != x->dtype || beta->dtype != x->dtype)
    return fail(TCAB_ERR_DTYPE, "%s: gamma, beta and y must have the element type of x", op);
  if (!same_shape(x, y)) return fail(TCAB_ERR_SHAPE, "%s: y must have the shape of x", op);
  const uint32_t cols = x->dims[x->rank - 1];
  if (gamma->rank != 1 || gamma->dims[0] != cols)
    return fail(TCAB_ERR_SHAPE, "%s: gamma must be rank 1 with extent %u (the innermost extent of x)", op, cols);
  if (beta->rank != 1 || beta->dims[0] != cols)
    return fail(TCAB_ERR_SHAPE, "%s: beta must be rank 1 with extent %u (the innermost extent of x)", op, cols);
  const unsigned es = x->dtype == TCAB_F32 ? 4 : 2;
  TCAB_TRY(need_elem_align(op, "x", x, es));
  TCAB_TRY(need_elem_align(op, "y", y, es));
  TCAB_TRY(need_elem_align(op, "gamma", gamma, es));
  TCAB_TRY(need_elem_align(op, "beta", beta, es));
  TCAB_TRY(have_device(op));
  const uint64_t rows = count(x, 0, x->rank - 1);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (x->dtype == TCAB_BF16)
    return launch_layernorm_rows_bf16(static_cast<const __nv_bfloat16*>(x->data),
                                      static_cast<const __nv_bfloat16*>(gamma->data),
                                      static_cast<const __nv_bfloat16*>(beta->data), eps,
                                      static_cast<__nv_bfloat16*>(y->data), rows, cols, s);
  return launch_layernorm_rows_f32(static_cast<const float*>(x->data), static_cast<const float*>(gamma->data),
                                   static_cast<const float*>(beta->data), eps, static_cast<float*>(y->data), rows,
                                   cols, s);
}

int tcab_reduce_outer(const tcab_tensor* t, const tcab_tensor* sum, const tcab_tensor* max,
                      const tcab_tensor* argmax, void* stream) {
  const char* op = "reduce_outer";
  TCAB_TRY(check_tensor(op, "t", t));
  TCAB_TRY(need_dtype(op, "t", t, TCAB_F32, "f32"));
  if (t->rank != 3) return fail(TCAB_ERR_SHAPE, "%s: t must be rank 3 [b, k, c]", op);
  if (sum == nullptr && max == nullptr && argmax == nullptr)
    return fail(TCAB_ERR_INVALID_ARG, "%s: at least one of sum, max, argmax is required", op);
  const tcab_tensor* outs[3] = {sum, max, argmax};
  const char* names[3] = {"sum", "max", "argmax"};
  for (int i = 0; i < 3; ++i) {
    if (outs[i] == nullptr) continue;
    TCAB_TRY(check_tensor(op, names[i], outs[i]));
    TCAB_TRY(need_dtype(op, names[i], outs[i], i == 2 ? TCAB_I32 : TCAB_F32, i == 2 ? "i32" : "f32"));
    if (outs[i]->rank != 2 || outs[i]->dims[0] != t->dims[0] || outs[i]->dims[1] != t->dims[2])
      return fail(TCAB_ERR_SHAPE, "%s: %s must be [%u, %u]", op, names[i], t->dims[0], t->dims[2]);
    TCAB_TRY(need_elem_align(op, names[i], outs[i], 4));
  }
  TCAB_TRY(need_elem_align(op, "t", t, 4));
  TCAB_TRY(have_device(op));
  return launch_reduce_outer(static_cast<const float*>(t->data), sum ? static_cast<float*>(sum->data) : nullptr,
                             max ? static_cast<float*>(max->data) : nullptr,
                             argmax ? static_cast<int32_t*>(argmax->data) : nullptr, t->dims[0], t->dims[1],
                             t->dims[2], static_cast<cudaStream_t>(stream));
}

int tcab_chain_reduce(const tcab_chain* chain, const tcab_tensor* ins, uint32_t n_ins, uint32_t reduce_axis,
                      const tcab_tensor* out, void* stream) {
  const char* op = "chain_reduce";
  if (chain == nullptr || chain->map_expr == nullptr || chain->combine_expr == nullptr)
    return fail(TCAB_ERR_INVALID_ARG, "%s: chain, map_expr and combine_expr are required", op);
  if (chain->n_captures > TCAB_MAX_CAPTURES)
    return fail(TCAB_ERR_INVALID_ARG, "%s: %u captures (at most %d)", op, chain->n_captures, TCAB_MAX_CAPTURES);
  if (ins == nullptr || n_ins < 1 || n_ins > TCAB_MAX_INPUTS)
    return fail(TCAB_ERR_INVALID_ARG, "%s: between 1 and %d operands are required", op, TCAB_MAX_INPUTS);
  const float* ptrs[TCAB_MAX_INPUTS] = {};
  int types[TCAB_MAX_INPUTS] = {};  // TCAB_F32 == 0
  for (uint32_t i = 0; i < n_ins; ++i) {
    char name[16];
    std::snprintf(name, sizeof(name), "ins[%u]", i);
    TCAB_TRY(check_tensor(op, name, &ins[i]));
    TCAB_TRY(need_operand_dtype(op, name, &ins[i]));
    if (ins[i].rank != ins[0].rank) return fail(TCAB_ERR_SHAPE, "%s: %s must have the rank of ins[0]", op, name);
    ptrs[i] = static_cast<const float*>(ins[i].data);
    types[i] = ins[i].dtype;
  }
  // the iteration shape: per axis the largest extent among the operands; an operand may have extent 1 along the
  // innermost axis (one value per row) or along every other axis (one row shared by all rows)
  tcab_tensor full = ins[0];
  for (uint32_t i = 1; i < n_ins; ++i)
    for (uint32_t d = 0; d < full.rank; ++d)
      if (ins[i].dims[d] > full.dims[d]) full.dims[d] = ins[i].dims[d];
  if (reduce_axis >= full.rank) return fail(TCAB_ERR_INVALID_ARG, "%s: reduce_axis %u out of range", op, reduce_axis);
  int rb = 0, cb = 0, cells = 0;
  for (uint32_t i = 0; i < n_ins; ++i) {
    int how = operand_indexing(full.dims, full.rank, &ins[i]);
    if (how != 0 && reduce_axis != full.rank - 1) {
      // a middle-axis reduction: an operand may lack the REDUCED axis (extent 1 there, the common extents elsewhere):
      // one value per output cell
      bool cell = ins[i].dims[reduce_axis] == 1;
      for (uint32_t d = 0; cell && d < full.rank; ++d) cell = d == reduce_axis || ins[i].dims[d] == full.dims[d];
      if (!cell)
        return fail(TCAB_ERR_SHAPE, "%s: ins[%u] must have the operands' common shape, or extent 1 along the reduced axis", op, i);
      cells |= 1 << i;
      continue;
    }
    if (how < 0)
      return fail(TCAB_ERR_SHAPE, "%s: ins[%u] must have the operands' common shape, or extent 1 along the innermost axis, "
                  "or extent 1 along every other axis", op, i);
    rb |= (how == 1) << i;
    cb |= (how == 2) << i;
  }
  const tcab_tensor* t = &full;
  TCAB_TRY(check_tensor(op, "out", out));
  TCAB_TRY(need_dtype(op, "out", out, TCAB_F32, "f32"));
  TCAB_TRY(need_elem_align(op, "out", out, 4));
  // out = the operands' extents minus the reduced axis (rank 1 -> [1]).
  uint32_t want[TCAB_MAX_RANK], wr = 0;
  for (uint32_t i = 0; i < t->rank; ++i)
    if (i != reduce_axis) want[wr++] = t->dims[i];
  if (wr == 0) want[wr++] = 1;
  bool ok = out->rank == wr;
  for (uint32_t i = 0; ok && i < wr; ++i) ok = out->dims[i] == want[i];
  if (!ok) return fail(TCAB_ERR_SHAPE, "%s: out must have the operands' extents without axis %u", op, reduce_axis);
  PreparedChain pc;
  TCAB_TRY(prepare_chain(chain, n_ins, &pc, 'R', types, TCAB_F32, rb, cb, cells));
  TCAB_TRY(have_device(op));
  return launch_chain_reduce(pc, ptrs, count(t, 0, reduce_axis), t->dims[reduce_axis],
                             count(t, reduce_axis + 1, t->rank), static_cast<float*>(out->data),
                             static_cast<cudaStream_t>(stream));
}

int tcab_chain_reduce_batched(const tcab_chain* chain, const tcab_tensor* ins, uint32_t n_ins, uint32_t n_problems,
                              const tcab_tensor* outs, void* stream) {
  const char* op = "chain_reduce_batched";
  if (chain == nullptr || chain->map_expr == nullptr || chain->combine_expr == nullptr)
    return fail(TCAB_ERR_INVALID_ARG, "%s: chain, map_expr and combine_expr are required", op);
  if (chain->n_captures > TCAB_MAX_CAPTURES)
    return fail(TCAB_ERR_INVALID_ARG, "%s: %u captures (at most %d)", op, chain->n_captures, TCAB_MAX_CAPTURES);
  if (ins == nullptr || outs == nullptr || n_ins < 1 || n_ins > TCAB_MAX_INPUTS)
    return fail(TCAB_ERR_INVALID_ARG, "%s: between 1 and %d operands per problem are required", op, TCAB_MAX_INPUTS);
  if (n_problems < 1 || n_problems > TCAB_MAX_BATCH)
    return fail(TCAB_ERR_TOO_LARGE, "%s: %u problems (between 1 and %d per call)", op, n_problems, TCAB_MAX_BATCH);
  const float* ptrs[TCAB_MAX_BATCH * TCAB_MAX_INPUTS] = {};
  float* optrs[TCAB_MAX_BATCH] = {};
  int types[TCAB_MAX_INPUTS] = {};  // TCAB_F32 == 0
  const tcab_tensor* t0 = &ins[0];
  for (uint32_t b = 0; b < n_problems; ++b) {
    for (uint32_t i = 0; i < n_ins; ++i) {
      const tcab_tensor* t = &ins[b * n_ins + i];
      char name[32];
      std::snprintf(name, sizeof(name), "ins[%u][%u]", b, i);
      TCAB_TRY(check_tensor(op, name, t));
      TCAB_TRY(need_operand_dtype(op, name, t));
      if (!same_shape(t0, t)) return fail(TCAB_ERR_SHAPE, "%s: %s must have the shape of ins[0][0]", op, name);
      if (b == 0) types[i] = t->dtype;
      else if (t->dtype != types[i]) return fail(TCAB_ERR_DTYPE, "%s: %s must have the element type of ins[0][%u]", op, name, i);
      ptrs[b * n_ins + i] = static_cast<const float*>(t->data);
    }
    const tcab_tensor* o = &outs[b];
    char name[32];
    std::snprintf(name, sizeof(name), "outs[%u]", b);
    TCAB_TRY(check_tensor(op, name, o));
    TCAB_TRY(need_dtype(op, name, o, TCAB_F32, "f32"));
    TCAB_TRY(need_elem_align(op, name, o, 4));
    bool ok = t0->rank == 1 ? (o->rank == 1 && o->dims[0] == 1) : o->rank == t0->rank - 1;
    for (uint32_t i = 0; ok && t0->rank > 1 && i + 1 < t0->rank; ++i) ok = o->dims[i] == t0->dims[i];
    if (!ok) return fail(TCAB_ERR_SHAPE, "%s: %s must have the operands' extents without the innermost axis", op, name);
    optrs[b] = static_cast<float*>(o->data);
  }
  PreparedChain pc;
  TCAB_TRY(prepare_chain(chain, n_ins, &pc, 'R', types));
  TCAB_TRY(have_device(op));
  return launch_chain_reduce_batched(pc, ptrs, optrs, n_problems, static_cast<uint32_t>(count(t0, 0, t0->rank - 1)),
                                     t0->dims[t0->rank - 1], static_cast<cudaStream_t>(stream));
}

int tcab_chain_reduce_noalloc(const tcab_chain* chain, const tcab_tensor* ins, uint32_t n_ins,
                              const tcab_tensor* out, void* stream) {
  const char* op = "chain_reduce_noalloc";
  if (chain == nullptr || chain->map_expr == nullptr || chain->combine_expr == nullptr)
    return fail(TCAB_ERR_INVALID_ARG, "%s: chain, map_expr and combine_expr are required", op);
  if (chain->n_captures > TCAB_MAX_CAPTURES)
    return fail(TCAB_ERR_INVALID_ARG, "%s: %u captures (at most %d)", op, chain->n_captures, TCAB_MAX_CAPTURES);
  if (ins == nullptr || n_ins < 1 || n_ins > TCAB_MAX_INPUTS)
    return fail(TCAB_ERR_INVALID_ARG, "%s: between 1 and %d operands are required", op, TCAB_MAX_INPUTS);
  const float* ptrs[TCAB_MAX_INPUTS] = {};
  int types[TCAB_MAX_INPUTS] = {};  // TCAB_F32 == 0
  for (uint32_t i = 0; i < n_ins; ++i) {
    char name[16];
    std::snprintf(name, sizeof(name), "ins[%u]", i);
    TCAB_TRY(check_tensor(op, name, &ins[i]));
    TCAB_TRY(need_operand_dtype(op, name, &ins[i]));
    if (i > 0 && !same_shape(&ins[0], &ins[i]))
      return fail(TCAB_ERR_SHAPE, "%s: %s must have the shape of ins[0]", op, name);
    ptrs[i] = static_cast<const float*>(ins[i].data);
    types[i] = ins[i].dtype;
  }
  const tcab_tensor* t = &ins[0];
  TCAB_TRY(check_tensor(op, "out", out));
  TCAB_TRY(need_dtype(op, "out", out, TCAB_F32, "f32"));
  TCAB_TRY(need_elem_align(op, "out", out, 4));
  const uint64_t rows = count(t, 0, t->rank - 1);
  bool ok = t->rank == 1 ? (out->rank == 1 && out->dims[0] == 1) : out->rank == t->rank - 1;
  for (uint32_t i = 0; ok && t->rank > 1 && i + 1 < t->rank; ++i) ok = out->dims[i] == t->dims[i];
  if (!ok) return fail(TCAB_ERR_SHAPE, "%s: out must have the operands' extents without the innermost axis", op);
  if (rows > TCAB_NOALLOC_MAX_ROWS)
    return fail(TCAB_ERR_TOO_LARGE,
                "%s: %llu rows exceed TCAB_NOALLOC_MAX_ROWS = %d (the fixed scratch array); use tcab_chain_reduce",
                op, static_cast<unsigned long long>(rows), TCAB_NOALLOC_MAX_ROWS);
  PreparedChain pc;
  TCAB_TRY(prepare_chain(chain, n_ins, &pc, 'R', types));
  TCAB_TRY(have_device(op));
  return launch_chain_reduce_noalloc(pc, ptrs, rows, t->dims[t->rank - 1], static_cast<float*>(out->data),
                                     static_cast<cudaStream_t>(stream));
}

int tcab_map(const tcab_chain* chain, const tcab_tensor* ins, uint32_t n_ins, const tcab_tensor* out, void* stream) {
  const char* op = "map";
  if (chain == nullptr || chain->map_expr == nullptr) return fail(TCAB_ERR_INVALID_ARG, "%s: chain and map_expr are required", op);
  if (chain->n_captures > TCAB_MAX_CAPTURES)
    return fail(TCAB_ERR_INVALID_ARG, "%s: %u captures (at most %d)", op, chain->n_captures, TCAB_MAX_CAPTURES);
  if (ins == nullptr || n_ins < 1 || n_ins > TCAB_MAX_INPUTS)
    return fail(TCAB_ERR_INVALID_ARG, "%s: between 1 and %d operands are required", op, TCAB_MAX_INPUTS);
  TCAB_TRY(check_tensor(op, "out", out));
  TCAB_TRY(need_operand_dtype(op, "out", out));
  const void* ptrs[TCAB_MAX_INPUTS] = {};
  int types[TCAB_MAX_INPUTS] = {};  // TCAB_F32 == 0
  int rb = 0, cb = 0;
  for (uint32_t i = 0; i < n_ins; ++i) {
    char name[16];
    std::snprintf(name, sizeof(name), "ins[%u]", i);
    TCAB_TRY(check_tensor(op, name, &ins[i]));
    TCAB_TRY(need_operand_dtype(op, name, &ins[i]));
    const int how = operand_indexing(out->dims, out->rank, &ins[i]);
    if (how < 0)
      return fail(TCAB_ERR_SHAPE, "%s: %s must have the shape of out, or extent 1 along the innermost axis (one value per "
                  "row), or extent 1 along every other axis (one row shared by all rows)", op, name);
    rb |= (how == 1) << i;
    cb |= (how == 2) << i;
    ptrs[i] = ins[i].data;
    types[i] = ins[i].dtype;
  }
  PreparedChain pc;
  TCAB_TRY(prepare_chain(chain, n_ins, &pc, 'M', types, out->dtype, rb, cb));
  TCAB_TRY(have_device(op));
  return launch_chain_map(pc, ptrs, out->data, count(out, 0, out->rank), out->dims[out->rank - 1],
                          static_cast<cudaStream_t>(stream));
}

int tcab_chain_contract(const tcab_chain* chain, const tcab_tensor* lhs, const tcab_tensor* rhs, int rhs_is_nk,
                        const tcab_tensor* out, void* stream) {
  const char* op = "chain_contract";
  if (chain == nullptr || chain->map_expr == nullptr || chain->combine_expr == nullptr)
    return fail(TCAB_ERR_INVALID_ARG, "%s: chain, map_expr and combine_expr are required", op);
  if (chain->n_captures > TCAB_MAX_CAPTURES)
    return fail(TCAB_ERR_INVALID_ARG, "%s: %u captures (at most %d)", op, chain->n_captures, TCAB_MAX_CAPTURES);
  TCAB_TRY(check_tensor(op, "lhs", lhs));
  TCAB_TRY(check_tensor(op, "rhs", rhs));
  TCAB_TRY(check_tensor(op, "out", out));
  TCAB_TRY(need_operand_dtype(op, "lhs", lhs));
  TCAB_TRY(need_operand_dtype(op, "rhs", rhs));
  TCAB_TRY(need_dtype(op, "out", out, TCAB_F32, "f32"));
  if (lhs->rank != 2 || rhs->rank != 2 || out->rank != 2)
    return fail(TCAB_ERR_SHAPE, "%s: lhs, rhs and out must be rank 2", op);
  const uint32_t m = lhs->dims[0], k = lhs->dims[1];
  const uint32_t rk = rhs_is_nk ? rhs->dims[1] : rhs->dims[0], n = rhs_is_nk ? rhs->dims[0] : rhs->dims[1];
  if (rk != k) return fail(TCAB_ERR_SHAPE, "%s: rhs.Dim(%d) must equal lhs.Dim(1) (dim k)", op, rhs_is_nk ? 1 : 0);
  if (out->dims[0] != m || out->dims[1] != n) return fail(TCAB_ERR_SHAPE, "%s: out must be [%u, %u]", op, m, n);
  TCAB_TRY(need_elem_align(op, "out", out, 4));
  const int types[2] = {lhs->dtype, rhs->dtype};
  PreparedChain pc;
  TCAB_TRY(prepare_chain(chain, 2, &pc, 'C', types));
  TCAB_TRY(have_device(op));
  return launch_chain_contract(pc, static_cast<const float*>(lhs->data), static_cast<const float*>(rhs->data),
                               rhs_is_nk ? 1 : 0, static_cast<float*>(out->data), m, n, k,
                               static_cast<cudaStream_t>(stream));
}

int tcab_gemm_bias_act(const tcab_tensor* a, const tcab_tensor* b, const tcab_tensor* bias, int act,
                       const tcab_tensor* c, void* stream) {
  const char* op = "gemm_bias_act";
  TCAB_TRY(check_tensor(op, "a", a));
  TCAB_TRY(check_tensor(op, "b", b));
  TCAB_TRY(check_tensor(op, "c", c));
  TCAB_TRY(need_dtype(op, "a", a, TCAB_BF16, "bf16"));
  TCAB_TRY(need_dtype(op, "b", b, TCAB_BF16, "bf16"));
  TCAB_TRY(need_dtype(op, "c", c, TCAB_BF16, "bf16"));
  if (a->rank != 2 || b->rank != 2 || c->rank != 2) return fail(TCAB_ERR_SHAPE, "%s: a, b and c must be rank 2", op);
  const uint32_t m = a->dims[0], k = a->dims[1], n = b->dims[1];
  if (b->dims[0] != k) return fail(TCAB_ERR_SHAPE, "%s: b.Dim(0) must equal a.Dim(1) (dim k)", op);
  if (c->dims[0] != m || c->dims[1] != n) return fail(TCAB_ERR_SHAPE, "%s: c must be [%u, %u]", op, m, n);
  if (bias != nullptr) {
    TCAB_TRY(check_tensor(op, "bias", bias));
    TCAB_TRY(need_dtype(op, "bias", bias, TCAB_F32, "f32"));
    if (bias->rank != 1 || bias->dims[0] != n) return fail(TCAB_ERR_SHAPE, "%s: bias must be [%u]", op, n);
    TCAB_TRY(need_elem_align(op, "bias", bias, 4));
  }
  if (act != TCAB_ACT_NONE && act != TCAB_ACT_RELU) return fail(TCAB_ERR_INVALID_ARG, "%s: unknown activation %d", op, act);
  if (k % 8 != 0 || n % 8 != 0)
    return fail(TCAB_ERR_ALIGNMENT, "%s: K and N must be multiples of 8 (16-byte rows for the tensor maps)", op);
  TCAB_TRY(need_elem_align(op, "a", a, 16));
  TCAB_TRY(need_elem_align(op, "b", b, 16));
  TCAB_TRY(need_elem_align(op, "c", c, 16));
  TCAB_TRY(have_device(op));
  return launch_gemm_bias_act(static_cast<const __nv_bfloat16*>(a->data), static_cast<const __nv_bfloat16*>(b->data),
                              bias ? static_cast<const float*>(bias->data) : nullptr, act,
                              static_cast<__nv_bfloat16*>(c->data), m, n, k, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
