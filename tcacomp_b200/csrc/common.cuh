// common.cuh -- shared host and device helpers of the kernel library.
//
// Host side: status/error plumbing for the C ABI (the status-code replacement of
// the reference's TCA_REQUIRE / TCA_CUDA_CHECK exceptions, runtime/tca/check.h:18-44),
// per-device facts (SM count, opt-in shared memory -- the reference queries the
// latter per launch in ValidateLaunch, runtime/tca/launch.h:37-58; here it is
// queried once per device) and the launch counter.
// Device side: 128-bit streaming loads/stores and the shuffle / shared-memory
// reduction trees that replace the per-element WarpReducer brackets
// (runtime/tca/reducer.h:81-181) with ONE tree per row.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>

#include "../../include/tcab.h"

namespace tcab {

// ---------------------------------------------------------------------------
// host plumbing (defined in abi.cu)
// ---------------------------------------------------------------------------
int fail(int status, const char* fmt, ...);
void count_launch(unsigned n = 1);
int sm_count();             // SMs of the current device (cached per device)
int max_optin_smem();       // opt-in shared memory per block of the current device
int check_launch(const char* what);  // cudaGetLastError -> status

struct Tune {
  int p0 = 0, p1 = 0, p2 = 0, p3 = 0;
};
const Tune& tune(int family);
enum Family { kSoftmax = 0, kLayernorm = 1, kReduceInner = 2, kReduceOuter = 3, kGemm = 4, kFamilies = 5 };

// Resident CTAs per SM of a kernel at a block size / dynamic smem, cached per (function, block).
int occupancy(const void* fn, int block, size_t smem);

// Scratch memory the library owns: one buffer per (device, stream, kind), allocated with cudaMalloc the first
// time a launch on that stream needs it and kept until tcab_release_stream / tcab_release_all or process
// exit. Per stream, because launches on different streams may overlap on the GPU. Returns null when the
// allocation failed (the callers then take a path that needs no scratch). With `grow`, a buffer that is
// too small is freed (cudaFree synchronises the device, so nothing still reads it) and allocated anew.
// `zero`: the buffer is cleared when it is allocated (arrival counters that their users leave at zero).
enum ScratchKind { kScratchChainSplit = 0, kScratchOuter = 1, kScratchGemm = 2, kScratchGemmCounters = 3, kScratchSplit3 = 4, kScratchKinds = 5 };
void* stream_scratch(int kind, cudaStream_t stream, size_t bytes, bool grow, bool zero = false);

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

inline uint32_t pow2_ceil(uint32_t v) {
  uint32_t p = 1;
  while (p < v) p <<= 1;
  return p;
}

// Entry points of the operator classes (one .cu each).
int launch_softmax_rows(const float* x, float* y, uint64_t rows, uint32_t cols, cudaStream_t s);
// long rows held in shared memory (rows_smem.cu); the caller has checked 16-byte vectors and rows_smem_fits
bool rows_smem_fits(uint64_t row_bytes);
int rows_smem_status(int* out);
int launch_softmax_rows_smem(const float* x, float* y, uint64_t rows, uint32_t cols, cudaStream_t s);
int launch_layernorm_rows_smem_bf16(const __nv_bfloat16* x, const __nv_bfloat16* gamma, const __nv_bfloat16* beta,
                                    float eps, __nv_bfloat16* y, uint64_t rows, uint32_t cols, cudaStream_t s);
int launch_layernorm_rows_smem_f32(const float* x, const float* gamma, const float* beta, float eps, float* y,
                                   uint64_t rows, uint32_t cols, cudaStream_t s);
int launch_layernorm_rows_bf16(const __nv_bfloat16* x, const __nv_bfloat16* gamma,
                               const __nv_bfloat16* beta, float eps, __nv_bfloat16* y,
                               uint64_t rows, uint32_t cols, cudaStream_t s);
int launch_layernorm_rows_f32(const float* x, const float* gamma, const float* beta, float eps,
                              float* y, uint64_t rows, uint32_t cols, cudaStream_t s);
int launch_reduce_outer(const float* t, float* sum, float* mx, int32_t* amax, uint32_t nb,
                        uint32_t nk, uint32_t nc, cudaStream_t s);
// What the run-time compiler needs to know about a chain: which kernels ('R' the reduction kernels, 'B' the
// batched reduction kernels, 'C' the contraction kernels, 'M' the map-only kernels), the canonical lambdas and the element types.
struct JitSpec {
  char kind = 'R';
  int n_in = 0, combine = 0;
  int in_types[TCAB_MAX_INPUTS] = {};  // tcab_dtype of each operand (TCAB_F32 == 0)
  int out_type = TCAB_F32;                                                   // map-only: the stored element type
  int rb_mask = 0, cb_mask = 0;  // operands with one value per row / one row shared by all rows (innermost-axis kernels)
  int cell_mask = 0;             // middle-axis reductions: operands with one value per output cell (no reduced axis)
  std::string map_text, post_text;
  int bf_mask() const {
    int m = 0;
    for (int i = 0; i < n_in; ++i) m |= (in_types[i] == TCAB_BF16) << i;
    return m;
  }
};
// A chain whose lambdas were validated, canonicalised and matched to a compiled kernel.
struct PreparedChain {
  int entry = -1;   // index into the table of ahead-of-time chains, or kJitEntry
  float init = 0.0f;
  float caps[16];   // map captures in [0,8), piped-map captures in [8,16)
  JitSpec spec;     // canonical lambdas and types (always filled in)
};
constexpr int kJitEntry = -2;
// Run-time compilation of chains without an ahead-of-time instance (chain_jit.cu).
bool jit_available();
// Without compile_if_missing a chain that is not cached yet is TCAB_ERR_UNSUPPORTED.
int jit_prepare(const JitSpec& spec, void** handle, bool compile_if_missing = true);
int jit_compile_check(const JitSpec& spec);  // NVRTC only, nothing is loaded: works without a device
int jit_launch(void* handle, const float* const* ins, uint64_t outer, uint32_t nk, uint64_t inner, float init,
               const float* caps16, float* out, float* split_scratch_or_null, uint32_t splits, cudaStream_t s);
int jit_launch_map(void* handle, const void* const* ins, void* out, uint64_t n, uint32_t cols, const float* caps16,
                   cudaStream_t s);
// Host-only step (no device needed): parse, canonicalise and look the chain up.
// kind: 'R' / 'C' / 'M' as in JitSpec; in_types: n_ins tcab_dtype values (null = all f32); out_type: map-only.
int prepare_chain(const tcab_chain* chain, uint32_t n_ins, PreparedChain* pc, char kind = 'R', const int* in_types = nullptr,
                  int out_type = TCAB_F32, int rb_mask = 0, int cb_mask = 0, int cell_mask = 0);
int launch_chain_map(const PreparedChain& pc, const void* const* ins, void* out, uint64_t n, uint32_t cols, cudaStream_t s);
int launch_chain_reduce(const PreparedChain& pc, const float* const* ins, uint64_t outer, uint32_t nk,
                        uint64_t inner, float* out, cudaStream_t s);
int launch_gemm_bias_act(const __nv_bfloat16* a, const __nv_bfloat16* b, const float* bias,
                         int act, __nv_bfloat16* c, uint32_t m, uint32_t n, uint32_t k,
                         cudaStream_t s);

int launch_contract_bf16_tc(const __nv_bfloat16* a, const __nv_bfloat16* b, int b_is_nk, float alpha, float* c, uint32_t m,
                            uint32_t n, uint32_t k, cudaStream_t s, uint64_t c_pitch = 0);  // tensor cores, fp32 out (gemm_bias_act.cu)

// chain_outer_flat (a warp per (b, column tile)) instead of chain_outer (a CTA per tile) for a middle-axis
// reduction over [nb, nk, nc]. `vec`: 16-byte vectors (nc % 4 == 0, aligned operands: tiles of 128 columns, groups of
// four columns); otherwise 4-byte loads (tiles of 32 columns, groups of one). The warps take rows of at most 32
// columns, rows of up to 64 columns when there are many of them or few long ones, any row when the reduced axis is
// shorter than 64, and any row on 4-byte loads. Returns the column groups per tile (1..32), or 0 for a CTA per tile. Measured (fp32 sum over
// 2^28 elements, TB/s, a CTA per tile -> a warp per tile): [262144, 256, 4] 0.58 -> 7.1, [131072, 256, 8] 1.2 -> 6.9,
// [65536, 256, 16] 2.3 -> 6.9, [32768, 256, 32] 4.4 -> 6.9, [65536, 4, 1024] 1.6 -> 5.5, [131072, 8, 256] 2.6 ->
// 5.9, [262144, 16, 64] 2.6 -> 6.4; the fused sum / max / argmax kernel 0.36 -> 5.6, 0.73 -> 6.3, 1.4 -> 6.6, 2.7 ->
// 6.6 on the first four.
inline uint32_t outer_flat_width(uint32_t nc, bool vec) {  // the groups such a warp would use, whatever the rule says
  if (vec) return nc >= 128 ? 32u : nc / 4;
  return nc >= 32 ? 32u : nc;
}

inline uint32_t outer_flat_groups(uint64_t nb, uint32_t nk, uint32_t nc, int sm, bool vec) {
  if (nc == 0 || nk == 0 || (vec && nc % 4 != 0)) return 0;
  const uint32_t g = outer_flat_width(nc, vec);
  const uint32_t tile = vec ? 128u : 32u;
  const uint64_t work = nb * ((nc + tile - 1) / tile);  // warps
  // few long narrow columns (column statistics of a tall matrix): CTAs of these warps share the k axis, see
  // outer_flat_ranges; from a full tile on a CTA per tile already uses every lane
  if (work < 8ull * static_cast<uint64_t>(sm) && nk >= 1024) return nc <= tile / 2 ? g : 0;
  if (nc <= 32) return g;
  if (nk < 64) return g;
  // 4-byte loads: the warps are ahead on every shape measured ([128, 1024, 1022] 4.8 -> 5.8 TB/s, [4032, 256, 130]
  // 3.8 -> 5.6, [15887, 256, 33] 2.5 -> 4.9, [2052, 64, 1022] 3.6 -> 6.5)
  if (!vec) return g;
  // 36 ... 64 columns use at most half the lanes of a CTA's tile: the warps win only when there are enough of them to
  // keep an SM's memory pipeline full (measured [1024, 4096, 64]: 6.6 TB/s with a CTA per tile, 3.4 with 1024 warps)
  if (nc <= 64 && work >= 32ull * static_cast<uint64_t>(sm)) return g;
  return 0;
}

// The warp-per-tile kernels on few tiles and a long reduced axis: into how many ranges the k axis of one (b, column
// tile) is cut, a CTA of eight warps each -- eight CTAs per SM in total, every warp with at least 16 steps, within
// `max_partials` partial cells (one per range and output cell) -- and how many k rows a range has. 1 = no split.
// (Column statistics of a tall matrix, measured with CTAs of 128-column tiles sharing k: [1, 2^23, 16], where 16 of
// the 128 columns exist, 1.2 - 1.8 TB/s; [1, 2^25, 4]: 0.3 - 0.5.)
inline uint32_t outer_flat_ranges(uint64_t nb, uint32_t nk, uint32_t nc, uint32_t g, bool vec, int sm,
                                  uint64_t max_partials, uint32_t* klen) {
  const uint32_t tile = vec ? 128u : 32u;
  const uint64_t work = nb * ((nc + tile - 1) / tile), cells = nb * nc;
  const uint64_t target = 8ull * static_cast<uint64_t>(sm);
  uint64_t ranges = 1;
  if (work < target && cells > 0 && cells * 2 <= max_partials) {
    ranges = (target + work - 1) / work;
    const uint64_t rows_per_step = 32 / g, by_len = nk / (rows_per_step * 8 * 16);
    if (ranges > by_len) ranges = by_len;
    if (ranges > max_partials / cells) ranges = max_partials / cells;
    if (ranges < 2) ranges = 1;
  }
  uint32_t len = static_cast<uint32_t>((nk + ranges - 1) / ranges);
  ranges = (nk + len - 1) / len;  // no empty range
  *klen = len;
  return static_cast<uint32_t>(ranges);
}

// Threads that share the partials of one output of a split reduction in its finishing launch: a power of two that
// leaves each at most 16 of them.
inline uint32_t finish_lanes(uint32_t partials_per_out) {
  uint32_t lanes = 1;
  while (lanes < 32 && partials_per_out > 16 * lanes) lanes *= 2;
  return lanes;
}

// Innermost-axis chains: the row length (in vectors) from which a CTA of 256 threads takes a row instead of a warp.
inline uint32_t inner_cta_per_row_from(int n_in) { return n_in >= 2 ? 384u : 640u; }

// chain_inner_rows32: warps per CTA for rows of nvec vectors and n_in operands such that the CTA's shared memory
// stays within the 48 KiB that need no opt-in; 0 when not even one warp fits.
inline uint32_t rows32_warps(uint32_t nvec, int n_in) {
  const uint64_t per_warp = static_cast<uint64_t>(n_in) * 32 * (nvec + 1) * 16;
  const uint64_t w = per_warp ? (48 * 1024) / per_warp : 0;
  return w >= 8 ? 8u : static_cast<uint32_t>(w);
}

// chain_inner_rows32e (rows of nk elements that are not whole vectors): the same bound.
inline uint32_t rows32e_warps(uint32_t nk, int n_in) {
  const uint64_t per_warp = static_cast<uint64_t>(n_in) * 32 * nk * 4;
  const uint64_t w = per_warp ? (48 * 1024) / per_warp : 0;
  return w >= 8 ? 8u : static_cast<uint32_t>(w);
}

// fp32 operands, plain product: each operand is cut into three bf16 pieces and the six significant piece products
// run as ONE bf16 tensor-core contraction over 6 K. Returns TCAB_ERR_UNSUPPORTED (without a message) when the shape
// does not qualify or the workspace would exceed its cap: the caller keeps the scalar kernel.
int launch_contract_f32_split3(const float* a, const float* b, int b_is_nk, float alpha, float* c, uint32_t m, uint32_t n,
                               uint32_t k, cudaStream_t s);

int warm_chain(const PreparedChain& pc);  // compile + load now what a launch would compile later
int launch_chain_reduce_batched(const PreparedChain& pc, const float* const* ins, float* const* outs, uint32_t nprob,
                                uint32_t rows, uint32_t nk, cudaStream_t s);  // ins: [nprob][n_in]
int jit_launch_batched(void* handle, const float* const* ins, float* const* outs, uint32_t nprob, uint32_t rows, uint32_t nk,
                       float init, const float* caps16, cudaStream_t s);
int launch_chain_reduce_noalloc(const PreparedChain& pc, const float* const* ins, uint64_t rows, uint32_t nk,
                                float* out, cudaStream_t s);
int jit_launch_contract(void* handle, const float* lhs, const float* rhs, int rhs_nk, float* out, uint32_t m,
                        uint32_t n, uint32_t k, float init, const float* caps16, cudaStream_t s);
uint32_t choose_outer_splits(uint64_t tiles, uint64_t cells, uint32_t nk, uint64_t resident);  // chain_outer k ranges
uint32_t plan_outer_splits(uint64_t tiles, uint64_t cells, uint32_t nk, uint64_t resident, int sms, int forced);
bool inner_wants_big_ctas(uint64_t rows);  // chain_inner: 1024-thread CTAs for problems whose CTAs are all resident at once
void plan_outer_ranges(uint32_t wanted, uint32_t nk, uint32_t* ranges, uint32_t* klen);  // ranges that cover [0, nk), none empty
bool contract_big_tiles(uint32_t m, uint32_t n);  // tile choice of the fp32 contraction (tune "gemm" p2 = 4 / 8 forces it)
int launch_chain_contract(const PreparedChain& pc, const float* lhs, const float* rhs, int rhs_nk, float* out,
                          uint32_t m, uint32_t n, uint32_t k, cudaStream_t s);
int gemm_device_status(int* out);  // status word of the contraction kernel (synchronous read)

// ---------------------------------------------------------------------------
// device helpers
// ---------------------------------------------------------------------------
#ifdef __CUDACC__

constexpr unsigned kFullMask = 0xffffffffu;

// 128-bit loads/stores for data that is touched once. The cache policy is a build-time
// choice (TCAB_LD_POLICY / TCAB_ST_POLICY: 0 = evict-first "streaming", 1 = default,
// 2 = loads through the non-coherent path without L1 allocation).
#ifndef TCAB_LD_POLICY
#define TCAB_LD_POLICY 0
#endif
#ifndef TCAB_ST_POLICY
#define TCAB_ST_POLICY 0
#endif
__device__ __forceinline__ float4 ld_stream(const float4* p) {
#if TCAB_LD_POLICY == 0
  return __ldcs(p);
#elif TCAB_LD_POLICY == 1
  return *p;
#else
  float4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
  return v;
#endif
}
__device__ __forceinline__ uint4 ld_stream(const uint4* p) {
#if TCAB_LD_POLICY == 0
  return __ldcs(p);
#elif TCAB_LD_POLICY == 1
  return *p;
#else
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
#endif
}
__device__ __forceinline__ float ld_stream(const float* p) { return __ldcs(p); }
__device__ __forceinline__ void st_stream(float4* p, float4 v) {
#if TCAB_ST_POLICY == 0
  __stcs(p, v);
#else
  *p = v;
#endif
}
__device__ __forceinline__ void st_stream(uint4* p, uint4 v) {
#if TCAB_ST_POLICY == 0
  __stcs(p, v);
#else
  *p = v;
#endif
}
__device__ __forceinline__ void st_stream(float* p, float v) { __stcs(p, v); }

struct OpSum {
  static __device__ __forceinline__ float identity() { return 0.0f; }
  static __device__ __forceinline__ float apply(float a, float b) { return a + b; }
};
struct OpMax {
  static __device__ __forceinline__ float identity() { return -INFINITY; }
  static __device__ __forceinline__ float apply(float a, float b) { return fmaxf(a, b); }
};
struct OpMin {
  static __device__ __forceinline__ float identity() { return INFINITY; }
  static __device__ __forceinline__ float apply(float a, float b) { return fminf(a, b); }
};

// Butterfly over the low `WIDTH` lanes of each aligned lane group: every lane
// of the group ends with the group's result.
template <typename Op, int WIDTH = 32>
__device__ __forceinline__ float warp_allreduce(float v) {
#pragma unroll
  for (int off = WIDTH / 2; off > 0; off >>= 1) v = Op::apply(v, __shfl_xor_sync(kFullMask, v, off));
  return v;
}

// All `NWARPS` warps of the CTA combine one value each through `slots`
// (NWARPS floats of shared memory); every thread returns the result. ONE
// barrier: the caller alternates between two slot arrays so that a slot is
// never rewritten before every thread has read it (see the row kernels).
template <typename Op, int NWARPS>
__device__ __forceinline__ float cta_allreduce(float v, float* slots) {
  v = warp_allreduce<Op>(v);
  if constexpr (NWARPS == 1) {
    return v;
  } else {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) slots[warp] = v;
    __syncthreads();
    static_assert((NWARPS & (NWARPS - 1)) == 0 && NWARPS <= 32, "NWARPS must be a power of two");
    // Every aligned group of NWARPS lanes holds all the partials, so the
    // narrow butterfly leaves the full result in every lane.
    return warp_allreduce<Op, NWARPS>(slots[lane & (NWARPS - 1)]);
  }
}

// ---- thread-block clusters: distributed shared memory ---------------------------------------
__device__ __forceinline__ unsigned cluster_rank() {
  unsigned r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// Reads a float from the shared memory of CTA `rank` of this cluster, at the address that `local`
// has in this CTA (every CTA of a cluster lays its shared memory out identically).
__device__ __forceinline__ float ld_dsmem(const float* local, unsigned rank) {
  unsigned a = static_cast<unsigned>(__cvta_generic_to_shared(local)), ra;
  float v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(a), "r"(rank));
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(ra) : "memory");
  return v;
}
// All threads of all CTAs of the cluster: writes before the barrier are visible after it.
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

#endif  // __CUDACC__

}  // namespace tcab
