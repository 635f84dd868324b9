// pipeline.cu -- host-buffer execution behind the C ABI: upload, kernel and download pipelined over
// chunks of the independent axis, on one device (tcab_pipeline) or cut over several (tcab_multi).
//
// The reference's launchers take device tensors and leave the copies to the caller; its runners copy
// whole tensors around the launch (testing/runners/common.cuh:72-90: cudaMemcpy in, launch,
// synchronise, cudaMemcpy out), which serialises the two PCIe directions around the kernel. Every
// operator class here has an axis along which outputs are independent (rows / batch / rows of A), so
// the cut that shards a problem across GPUs also pipelines it on one GPU: chunk i+1 uploads while
// chunk i computes and chunk i-1 downloads.
//
// Three streams per pipeline, one per stage, so that neither copy direction ever queues behind a copy
// of the other direction; `depth` staging slots rotate; per slot three events order its stages
// (upload -> kernel -> download) and its reuse (the next upload into a slot waits for the kernel that
// read it, the next kernel for the download that read its outputs). Nothing here waits on the host
// except tcab_pipeline_sync / tcab_multi_sync.
#include <cstring>
#include <mutex>
#include <new>
#include <string>
#include <vector>

#include "common.cuh"

namespace tcab {
namespace {

size_t dtype_bytes(int dt) { return dt == TCAB_BF16 ? 2 : 4; }

struct Slot {
  void* in[TCAB_MAX_INPUTS] = {};
  void* out[TCAB_PIPELINE_MAX_OUTPUTS] = {};
  cudaEvent_t uploaded = nullptr, computed = nullptr, downloaded = nullptr;
  bool used = false;
};

struct OutSpec {
  int dtype = TCAB_F32;
  uint64_t unit_elems = 1;        // elements one unit of the independent axis produces
  uint32_t rank = 0;              // rank of one unit's output (0: a scalar per unit)
  uint32_t dims[TCAB_MAX_RANK - 1] = {};
};

}  // namespace
}  // namespace tcab

using namespace tcab;

struct tcab_pipeline {
  tcab_pipeline_desc d;
  std::string map_expr, combine_expr, post_expr;  // owned copies of the chain's lambdas
  tcab_chain chain;
  int device = 0;
  uint32_t depth = 4;
  uint64_t unit_elems = 1;  // elements of ONE streamed operand per unit
  uint32_t n_outs = 0;
  OutSpec outs[TCAB_PIPELINE_MAX_OUTPUTS];
  cudaStream_t up = nullptr, compute = nullptr, down = nullptr;
  std::vector<Slot> slots;
  uint64_t next_chunk = 0;
  std::mutex mu;
};

struct tcab_multi {
  std::vector<tcab_pipeline*> pipes;
};

namespace tcab {
namespace {

struct DeviceGuard {
  int prev = -1;
  bool ok = false;
  explicit DeviceGuard(int dev) {
    if (cudaGetDevice(&prev) != cudaSuccess) {
      cudaGetLastError();
      return;
    }
    ok = prev == dev || cudaSetDevice(dev) == cudaSuccess;
    if (!ok) cudaGetLastError();
  }
  ~DeviceGuard() {
    if (prev >= 0) cudaSetDevice(prev);
  }
};

int cuda_fail(const char* what, cudaError_t e) {
  cudaGetLastError();
  return fail(TCAB_ERR_CUDA, "pipeline: %s failed: %s", what, cudaGetErrorString(e));
}

#define PIPE_CUDA(expr)                                        \
  do {                                                         \
    const cudaError_t pipe_e_ = (expr);                        \
    if (pipe_e_ != cudaSuccess) return cuda_fail(#expr, pipe_e_); \
  } while (0)

// What one unit of the independent axis looks like on the output side, per operator class.
int plan_outputs(tcab_pipeline* p) {
  const tcab_pipeline_desc& d = p->d;
  const uint32_t last = d.unit_dims[d.unit_rank - 1];
  auto same_as_input = [&](int dtype) {
    OutSpec o;
    o.dtype = dtype;
    o.unit_elems = p->unit_elems;
    o.rank = d.unit_rank;
    for (uint32_t i = 0; i < d.unit_rank; ++i) o.dims[i] = d.unit_dims[i];
    return o;
  };
  switch (d.op) {
    case TCAB_OP_SOFTMAX_ROWS:
      if (d.in_dtype != TCAB_F32) return fail(TCAB_ERR_DTYPE, "pipeline: softmax rows are f32");
      p->outs[p->n_outs++] = same_as_input(TCAB_F32);
      return TCAB_OK;
    case TCAB_OP_LAYERNORM_ROWS:
      if (d.in_dtype != TCAB_F32 && d.in_dtype != TCAB_BF16) return fail(TCAB_ERR_DTYPE, "pipeline: layer-norm rows are f32 or bf16");
      if (d.resident[0].data == nullptr || d.resident[1].data == nullptr)
        return fail(TCAB_ERR_INVALID_ARG, "pipeline: layer-norm needs gamma and beta (device tensors) in resident[0], resident[1]");
      p->outs[p->n_outs++] = same_as_input(d.in_dtype);
      return TCAB_OK;
    case TCAB_OP_REDUCE_OUTER: {
      if (d.unit_rank != 2 || d.in_dtype != TCAB_F32)
        return fail(TCAB_ERR_SHAPE, "pipeline: reduce_outer streams f32 units of shape [k, c]");
      if ((d.outputs & 7u) == 0) return fail(TCAB_ERR_INVALID_ARG, "pipeline: reduce_outer needs outputs (bit 0 sum, 1 max, 2 argmax)");
      for (int i = 0; i < 3; ++i) {
        if (!(d.outputs & (1u << i))) continue;
        OutSpec o;
        o.dtype = i == 2 ? TCAB_I32 : TCAB_F32;
        o.unit_elems = last;
        o.rank = 1;
        o.dims[0] = last;
        p->outs[p->n_outs++] = o;
      }
      return TCAB_OK;
    }
    case TCAB_OP_CHAIN_REDUCE: {
      if (d.unit_rank != 1 || (d.in_dtype != TCAB_F32 && d.in_dtype != TCAB_BF16))
        return fail(TCAB_ERR_SHAPE, "pipeline: chain_reduce streams f32 or bf16 rows (unit rank 1), reduced along the row");
      if (d.chain == nullptr) return fail(TCAB_ERR_INVALID_ARG, "pipeline: chain_reduce needs a chain");
      OutSpec o;  // one scalar per row
      p->outs[p->n_outs++] = o;
      return TCAB_OK;
    }
    case TCAB_OP_GEMM_BIAS_ACT: {
      if (d.unit_rank != 1 || d.in_dtype != TCAB_BF16) return fail(TCAB_ERR_SHAPE, "pipeline: the contraction streams bf16 rows of a");
      const tcab_tensor& b = d.resident[0];
      if (b.data == nullptr || b.rank != 2 || b.dims[0] != last)
        return fail(TCAB_ERR_SHAPE, "pipeline: resident[0] must be b [K, N] on the device with K = the row length of a");
      OutSpec o;
      o.dtype = TCAB_BF16;
      o.unit_elems = b.dims[1];
      o.rank = 1;
      o.dims[0] = b.dims[1];
      p->outs[p->n_outs++] = o;
      return TCAB_OK;
    }
    case TCAB_OP_MAP: {
      if (d.chain == nullptr) return fail(TCAB_ERR_INVALID_ARG, "pipeline: map needs a chain (map_expr)");
      p->outs[p->n_outs++] = same_as_input(d.out_dtype);
      return TCAB_OK;
    }
    default:
      return fail(TCAB_ERR_INVALID_ARG, "pipeline: unknown operator %d", d.op);
  }
}

tcab_tensor chunk_view(void* data, int dtype, uint64_t n, uint32_t rank, const uint32_t* dims) {
  tcab_tensor t;
  std::memset(&t, 0, sizeof(t));
  t.data = data;
  t.dtype = dtype;
  t.rank = rank + 1;
  t.dims[0] = static_cast<uint32_t>(n);
  for (uint32_t i = 0; i < rank; ++i) t.dims[i + 1] = dims[i];
  return t;
}

// One launch of the pipeline's operator on n units held in a staging slot, on the compute stream.
int launch_chunk(tcab_pipeline* p, Slot& s, uint64_t n) {
  const tcab_pipeline_desc& d = p->d;
  tcab_tensor ins[TCAB_MAX_INPUTS];
  for (uint32_t i = 0; i < d.n_streamed; ++i) ins[i] = chunk_view(s.in[i], d.in_dtype, n, d.unit_rank, d.unit_dims);
  tcab_tensor outs[TCAB_PIPELINE_MAX_OUTPUTS];
  for (uint32_t i = 0; i < p->n_outs; ++i) {
    outs[i] = chunk_view(s.out[i], p->outs[i].dtype, n, p->outs[i].rank, p->outs[i].dims);
    if (p->outs[i].rank == 0) outs[i].rank = 1;  // a scalar per unit: [n]
  }
  switch (d.op) {
    case TCAB_OP_SOFTMAX_ROWS:
      return tcab_softmax_rows(&ins[0], &outs[0], p->compute);
    case TCAB_OP_LAYERNORM_ROWS:
      return tcab_layernorm_rows(&ins[0], &d.resident[0], &d.resident[1], d.eps, &outs[0], p->compute);
    case TCAB_OP_REDUCE_OUTER: {
      const tcab_tensor* o[3] = {nullptr, nullptr, nullptr};
      uint32_t k = 0;
      for (int i = 0; i < 3; ++i)
        if (d.outputs & (1u << i)) o[i] = &outs[k++];
      return tcab_reduce_outer(&ins[0], o[0], o[1], o[2], p->compute);
    }
    case TCAB_OP_CHAIN_REDUCE:
      return tcab_chain_reduce(&p->chain, ins, d.n_streamed, 1, &outs[0], p->compute);
    case TCAB_OP_GEMM_BIAS_ACT:
      return tcab_gemm_bias_act(&ins[0], &d.resident[0], d.resident[1].data ? &d.resident[1] : nullptr, d.act, &outs[0],
                                p->compute);
    case TCAB_OP_MAP:
      return tcab_map(&p->chain, ins, d.n_streamed, &outs[0], p->compute);
    default:
      return fail(TCAB_ERR_INVALID_ARG, "pipeline: unknown operator %d", d.op);
  }
}

void destroy_pipeline(tcab_pipeline* p) {
  if (p == nullptr) return;
  DeviceGuard g(p->device);
  if (p->down) cudaStreamSynchronize(p->down);
  if (p->compute) cudaStreamSynchronize(p->compute);
  if (p->up) cudaStreamSynchronize(p->up);
  for (Slot& s : p->slots) {
    for (void* q : s.in)
      if (q) cudaFree(q);
    for (void* q : s.out)
      if (q) cudaFree(q);
    if (s.uploaded) cudaEventDestroy(s.uploaded);
    if (s.computed) cudaEventDestroy(s.computed);
    if (s.downloaded) cudaEventDestroy(s.downloaded);
  }
  if (p->compute) tcab_release_stream(p->compute);  // scratch the kernels took for this stream
  if (p->up) cudaStreamDestroy(p->up);
  if (p->compute) cudaStreamDestroy(p->compute);
  if (p->down) cudaStreamDestroy(p->down);
  cudaGetLastError();
  delete p;
}

// Queues the three stages of one chunk: units [lo, hi) of the caller's host buffers.
int enqueue_chunk(tcab_pipeline* p, const void* const* host_ins, void* const* host_outs, uint64_t lo, uint64_t hi) {
  const tcab_pipeline_desc& d = p->d;
  Slot& s = p->slots[p->next_chunk % p->depth];
  ++p->next_chunk;
  const uint64_t n = hi - lo;
  const size_t in_unit = p->unit_elems * dtype_bytes(d.in_dtype);
  if (s.used) PIPE_CUDA(cudaStreamWaitEvent(p->up, s.computed, 0));  // the kernel that read this slot's input
  for (uint32_t i = 0; i < d.n_streamed; ++i)
    PIPE_CUDA(cudaMemcpyAsync(s.in[i], static_cast<const char*>(host_ins[i]) + lo * in_unit, n * in_unit,
                              cudaMemcpyHostToDevice, p->up));
  PIPE_CUDA(cudaEventRecord(s.uploaded, p->up));
  PIPE_CUDA(cudaStreamWaitEvent(p->compute, s.uploaded, 0));
  if (s.used) PIPE_CUDA(cudaStreamWaitEvent(p->compute, s.downloaded, 0));  // the download that read this slot's outputs
  const int rc = launch_chunk(p, s, n);
  if (rc != TCAB_OK) return rc;
  PIPE_CUDA(cudaEventRecord(s.computed, p->compute));
  PIPE_CUDA(cudaStreamWaitEvent(p->down, s.computed, 0));
  for (uint32_t i = 0; i < p->n_outs; ++i) {
    const size_t out_unit = p->outs[i].unit_elems * dtype_bytes(p->outs[i].dtype);
    PIPE_CUDA(cudaMemcpyAsync(static_cast<char*>(host_outs[i]) + lo * out_unit, s.out[i], n * out_unit,
                              cudaMemcpyDeviceToHost, p->down));
  }
  PIPE_CUDA(cudaEventRecord(s.downloaded, p->down));
  s.used = true;
  return TCAB_OK;
}

int check_run_args(const tcab_pipeline* p, const void* const* host_ins, void* const* host_outs) {
  if (p == nullptr || host_ins == nullptr || host_outs == nullptr) return fail(TCAB_ERR_INVALID_ARG, "pipeline_run: null argument");
  for (uint32_t i = 0; i < p->d.n_streamed; ++i)
    if (host_ins[i] == nullptr) return fail(TCAB_ERR_INVALID_ARG, "pipeline_run: host_ins[%u] is null", i);
  for (uint32_t i = 0; i < p->n_outs; ++i)
    if (host_outs[i] == nullptr) return fail(TCAB_ERR_INVALID_ARG, "pipeline_run: host_outs[%u] is null", i);
  return TCAB_OK;
}

}  // namespace
}  // namespace tcab

extern "C" {

int tcab_shard_block(uint64_t n, uint32_t world, uint32_t rank, uint64_t* lo, uint64_t* hi) {
  if (world < 1 || rank >= world || lo == nullptr || hi == nullptr)
    return fail(TCAB_ERR_INVALID_ARG, "shard_block: bad rank %u of %u", rank, world);
  const uint64_t base = n / world, extra = n % world;
  *lo = rank * base + (rank < extra ? rank : extra);
  *hi = *lo + base + (rank < extra ? 1 : 0);
  return TCAB_OK;
}

int tcab_host_alloc(uint64_t bytes, void** out) {
  if (out == nullptr) return fail(TCAB_ERR_INVALID_ARG, "host_alloc: null output");
  *out = nullptr;
  const cudaError_t e = cudaHostAlloc(out, bytes > 0 ? bytes : 1, cudaHostAllocPortable);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(TCAB_ERR_CUDA, "host_alloc: cudaHostAlloc of %llu bytes failed: %s", static_cast<unsigned long long>(bytes),
                cudaGetErrorString(e));
  }
  return TCAB_OK;
}

int tcab_host_free(void* p) {
  if (p == nullptr) return TCAB_OK;
  const cudaError_t e = cudaFreeHost(p);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(TCAB_ERR_CUDA, "host_free: %s", cudaGetErrorString(e));
  }
  return TCAB_OK;
}

int tcab_pipeline_create(const tcab_pipeline_desc* desc, tcab_pipeline** out) {
  if (desc == nullptr || out == nullptr) return fail(TCAB_ERR_INVALID_ARG, "pipeline_create: null argument");
  *out = nullptr;
  if (desc->unit_rank < 1 || desc->unit_rank > TCAB_MAX_RANK - 1)
    return fail(TCAB_ERR_INVALID_ARG, "pipeline_create: unit_rank %u outside 1..%d", desc->unit_rank, TCAB_MAX_RANK - 1);
  if (desc->chunk_units == 0) return fail(TCAB_ERR_INVALID_ARG, "pipeline_create: chunk_units must be positive");
  if (desc->n_streamed < 1 || desc->n_streamed > TCAB_MAX_INPUTS ||
      (desc->n_streamed != 1 && desc->op != TCAB_OP_CHAIN_REDUCE && desc->op != TCAB_OP_MAP))
    return fail(TCAB_ERR_INVALID_ARG, "pipeline_create: bad number of streamed operands %u", desc->n_streamed);
  if (desc->depth != 0 && (desc->depth < 2 || desc->depth > 8))
    return fail(TCAB_ERR_INVALID_ARG, "pipeline_create: depth %u outside 2..8", desc->depth);
  tcab_pipeline* p = new (std::nothrow) tcab_pipeline();
  if (p == nullptr) return fail(TCAB_ERR_INVALID_ARG, "pipeline_create: out of host memory");
  p->d = *desc;
  p->depth = desc->depth ? desc->depth : 4;
  std::memset(&p->chain, 0, sizeof(p->chain));
  if (desc->chain != nullptr) {  // the caller's strings need not outlive this call
    p->chain = *desc->chain;
    if (desc->chain->map_expr) p->map_expr = desc->chain->map_expr;
    if (desc->chain->combine_expr) p->combine_expr = desc->chain->combine_expr;
    if (desc->chain->post_expr) p->post_expr = desc->chain->post_expr;
    p->chain.map_expr = desc->chain->map_expr ? p->map_expr.c_str() : nullptr;
    p->chain.combine_expr = desc->chain->combine_expr ? p->combine_expr.c_str() : nullptr;
    p->chain.post_expr = desc->chain->post_expr ? p->post_expr.c_str() : nullptr;
    p->d.chain = &p->chain;
  }
  p->unit_elems = 1;
  for (uint32_t i = 0; i < desc->unit_rank; ++i) p->unit_elems *= desc->unit_dims[i];
  if (p->unit_elems == 0 || p->unit_elems * desc->chunk_units >= (1ull << 32)) {
    delete p;
    return fail(TCAB_ERR_TOO_LARGE, "pipeline_create: a chunk must hold between 1 and 2^32 - 1 elements");
  }
  int rc = plan_outputs(p);
  if (rc != TCAB_OK) {
    delete p;
    return rc;
  }
  int dev = desc->device;
  if (dev < 0 && cudaGetDevice(&dev) != cudaSuccess) {
    cudaGetLastError();
    delete p;
    return fail(TCAB_ERR_CUDA, "pipeline_create: no CUDA device (this library has no CPU path)");
  }
  p->device = dev;
  DeviceGuard g(dev);
  if (!g.ok) {
    delete p;
    return fail(TCAB_ERR_CUDA, "pipeline_create: cannot select device %d", dev);
  }
  auto bail = [&](const char* what, cudaError_t e) {
    destroy_pipeline(p);
    return cuda_fail(what, e);
  };
  cudaError_t e;
  if ((e = cudaStreamCreateWithFlags(&p->up, cudaStreamNonBlocking)) != cudaSuccess) return bail("cudaStreamCreate", e);
  if ((e = cudaStreamCreateWithFlags(&p->compute, cudaStreamNonBlocking)) != cudaSuccess) return bail("cudaStreamCreate", e);
  if ((e = cudaStreamCreateWithFlags(&p->down, cudaStreamNonBlocking)) != cudaSuccess) return bail("cudaStreamCreate", e);
  p->slots.resize(p->depth);
  const size_t in_bytes = p->unit_elems * desc->chunk_units * dtype_bytes(desc->in_dtype);
  for (Slot& s : p->slots) {
    for (uint32_t i = 0; i < desc->n_streamed; ++i)
      if ((e = cudaMalloc(&s.in[i], in_bytes)) != cudaSuccess) return bail("cudaMalloc (input staging)", e);
    for (uint32_t i = 0; i < p->n_outs; ++i) {
      const size_t ob = p->outs[i].unit_elems * desc->chunk_units * dtype_bytes(p->outs[i].dtype);
      if ((e = cudaMalloc(&s.out[i], ob)) != cudaSuccess) return bail("cudaMalloc (output staging)", e);
    }
    if ((e = cudaEventCreateWithFlags(&s.uploaded, cudaEventDisableTiming)) != cudaSuccess) return bail("cudaEventCreate", e);
    if ((e = cudaEventCreateWithFlags(&s.computed, cudaEventDisableTiming)) != cudaSuccess) return bail("cudaEventCreate", e);
    if ((e = cudaEventCreateWithFlags(&s.downloaded, cudaEventDisableTiming)) != cudaSuccess) return bail("cudaEventCreate", e);
  }
  *out = p;
  return TCAB_OK;
}

uint32_t tcab_pipeline_outputs(const tcab_pipeline* p) { return p ? p->n_outs : 0; }

int tcab_pipeline_order_after(tcab_pipeline* p, void* stream) {
  if (p == nullptr) return fail(TCAB_ERR_INVALID_ARG, "pipeline_order_after: null pipeline");
  std::lock_guard<std::mutex> lk(p->mu);
  DeviceGuard g(p->device);
  if (!g.ok) return fail(TCAB_ERR_CUDA, "pipeline: cannot select device %d", p->device);
  cudaEvent_t ev;
  PIPE_CUDA(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
  cudaError_t e = cudaEventRecord(ev, static_cast<cudaStream_t>(stream));
  for (cudaStream_t s : {p->up, p->compute, p->down})
    if (e == cudaSuccess) e = cudaStreamWaitEvent(s, ev, 0);
  cudaEventDestroy(ev);  // released once the waits that reference it have completed
  if (e != cudaSuccess) return cuda_fail("ordering the pipeline after a stream", e);
  return TCAB_OK;
}

int tcab_pipeline_run(tcab_pipeline* p, const void* const* host_ins, uint64_t units, void* const* host_outs) {
  const int rc0 = check_run_args(p, host_ins, host_outs);
  if (rc0 != TCAB_OK) return rc0;
  std::lock_guard<std::mutex> lk(p->mu);
  DeviceGuard g(p->device);
  if (!g.ok) return fail(TCAB_ERR_CUDA, "pipeline: cannot select device %d", p->device);
  for (uint64_t lo = 0; lo < units; lo += p->d.chunk_units) {
    const uint64_t hi = lo + p->d.chunk_units < units ? lo + p->d.chunk_units : units;
    const int rc = enqueue_chunk(p, host_ins, host_outs, lo, hi);
    if (rc != TCAB_OK) return rc;
  }
  return TCAB_OK;
}

int tcab_pipeline_join(tcab_pipeline* p, void* stream) {
  if (p == nullptr) return fail(TCAB_ERR_INVALID_ARG, "pipeline_join: null pipeline");
  std::lock_guard<std::mutex> lk(p->mu);
  DeviceGuard g(p->device);
  if (!g.ok) return fail(TCAB_ERR_CUDA, "pipeline: cannot select device %d", p->device);
  // downloads are queued in chunk order behind their kernels and uploads: the end of the download stream is the end of the job
  cudaEvent_t ev;
  PIPE_CUDA(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
  cudaError_t e = cudaEventRecord(ev, p->down);
  if (e == cudaSuccess) e = cudaStreamWaitEvent(static_cast<cudaStream_t>(stream), ev, 0);
  cudaEventDestroy(ev);
  if (e != cudaSuccess) return cuda_fail("joining the pipeline", e);
  return TCAB_OK;
}

int tcab_pipeline_sync(tcab_pipeline* p) {
  if (p == nullptr) return fail(TCAB_ERR_INVALID_ARG, "pipeline_sync: null pipeline");
  DeviceGuard g(p->device);
  if (!g.ok) return fail(TCAB_ERR_CUDA, "pipeline: cannot select device %d", p->device);
  PIPE_CUDA(cudaStreamSynchronize(p->down));
  return TCAB_OK;
}

int tcab_pipeline_destroy(tcab_pipeline* p) {
  destroy_pipeline(p);
  return TCAB_OK;
}

// ---- one problem cut over several devices -----------------------------------------------------------

int tcab_multi_create(const tcab_pipeline_desc* descs, uint32_t n_devices, tcab_multi** out) {
  if (descs == nullptr || out == nullptr || n_devices < 1 || n_devices > 64)
    return fail(TCAB_ERR_INVALID_ARG, "multi_create: between 1 and 64 pipeline descriptions are required");
  *out = nullptr;
  for (uint32_t i = 0; i < n_devices; ++i) {
    if (descs[i].device < 0) return fail(TCAB_ERR_INVALID_ARG, "multi_create: descs[%u].device must name a device", i);
    for (uint32_t j = 0; j < i; ++j)
      if (descs[j].device == descs[i].device)
        return fail(TCAB_ERR_INVALID_ARG, "multi_create: device %d is named twice", descs[i].device);
    if (descs[i].op != descs[0].op || descs[i].unit_rank != descs[0].unit_rank || descs[i].in_dtype != descs[0].in_dtype ||
        descs[i].n_streamed != descs[0].n_streamed || descs[i].outputs != descs[0].outputs ||
        std::memcmp(descs[i].unit_dims, descs[0].unit_dims, sizeof(descs[0].unit_dims)) != 0)
      return fail(TCAB_ERR_SHAPE, "multi_create: descs[%u] describes a different operator or unit shape than descs[0]", i);
  }
  tcab_multi* m = new (std::nothrow) tcab_multi();
  if (m == nullptr) return fail(TCAB_ERR_INVALID_ARG, "multi_create: out of host memory");
  for (uint32_t i = 0; i < n_devices; ++i) {
    tcab_pipeline* p = nullptr;
    const int rc = tcab_pipeline_create(&descs[i], &p);
    if (rc != TCAB_OK) {
      for (tcab_pipeline* q : m->pipes) destroy_pipeline(q);
      delete m;
      return rc;
    }
    m->pipes.push_back(p);
  }
  *out = m;
  return TCAB_OK;
}

int tcab_multi_run(tcab_multi* m, const void* const* host_ins, uint64_t units, void* const* host_outs) {
  if (m == nullptr || m->pipes.empty()) return fail(TCAB_ERR_INVALID_ARG, "multi_run: null handle");
  const int rc0 = check_run_args(m->pipes[0], host_ins, host_outs);
  if (rc0 != TCAB_OK) return rc0;
  const uint32_t world = static_cast<uint32_t>(m->pipes.size());
  // device r owns the contiguous block tcab_shard_block(units, world, r); chunks are queued round-robin over
  // the devices so that all of them start at once
  std::vector<uint64_t> lo(world), hi(world);
  for (uint32_t r = 0; r < world; ++r) tcab_shard_block(units, world, r, &lo[r], &hi[r]);
  for (bool more = true; more;) {
    more = false;
    for (uint32_t r = 0; r < world; ++r) {
      if (lo[r] >= hi[r]) continue;
      tcab_pipeline* p = m->pipes[r];
      const uint64_t end = lo[r] + p->d.chunk_units < hi[r] ? lo[r] + p->d.chunk_units : hi[r];
      std::lock_guard<std::mutex> lk(p->mu);
      DeviceGuard g(p->device);
      if (!g.ok) return fail(TCAB_ERR_CUDA, "multi_run: cannot select device %d", p->device);
      const int rc = enqueue_chunk(p, host_ins, host_outs, lo[r], end);
      if (rc != TCAB_OK) return rc;
      lo[r] = end;
      more = more || lo[r] < hi[r];
    }
  }
  return TCAB_OK;
}

int tcab_multi_sync(tcab_multi* m) {
  if (m == nullptr) return fail(TCAB_ERR_INVALID_ARG, "multi_sync: null handle");
  for (tcab_pipeline* p : m->pipes) {
    const int rc = tcab_pipeline_sync(p);
    if (rc != TCAB_OK) return rc;
  }
  return TCAB_OK;
}

int tcab_multi_destroy(tcab_multi* m) {
  if (m == nullptr) return TCAB_OK;
  for (tcab_pipeline* p : m->pipes) destroy_pipeline(p);
  delete m;
  return TCAB_OK;
}

}  // extern "C"
