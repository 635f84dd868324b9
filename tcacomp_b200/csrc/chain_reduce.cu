// chain_reduce.cu -- ahead-of-time instances of the chain kernels and their dispatch.
//
// A chain arrives as canonical lambda text (expr.h). The table below holds the
// lambdas this build has compiled ahead of time, written as the same text the
// canonicaliser prints, so that the key and the code cannot drift apart: the
// macro stringifies the expression it compiles. A chain whose lambdas are not in
// the table is reported as unsupported by this build.
#include <mutex>
#include <string>
#include <utility>
#include <vector>

#include "chain_kernels.cuh"
#include "common.cuh"
#include "expr.h"

namespace tcab {
namespace {

using tcabk::Caps;
using tcabk::Ptrs;

// A lambda as device code: p0..p3 are the operands, c0..c7 the captures.
#define TCAB_LAMBDA(NAME, NIN, ...)                                                           \
  struct NAME {                                                                               \
    static constexpr int kIn = NIN;                                                           \
    static const char* text() { return #__VA_ARGS__; }                                        \
    static __device__ __forceinline__ float apply(const float* p, const float* c) {           \
      const float p0 = p[0], p1 = p[NIN > 1 ? 1 : 0], p2 = p[NIN > 2 ? 2 : 0], p3 = p[NIN > 3 ? 3 : 0]; \
      const float c0 = c[0], c1 = c[1], c2 = c[2], c3 = c[3], c4 = c[4], c5 = c[5], c6 = c[6], c7 = c[7]; \
      (void)p0; (void)p1; (void)p2; (void)p3;                                                 \
      (void)c0; (void)c1; (void)c2; (void)c3; (void)c4; (void)c5; (void)c6; (void)c7;         \
      return __VA_ARGS__;                                                                     \
    }                                                                                         \
  };

TCAB_LAMBDA(MapIdent, 1, p0)
TCAB_LAMBDA(MapAffineSq, 1, (((c0 * p0) + c1) * ((c0 * p0) + c1)))
TCAB_LAMBDA(MapMul2, 2, (p0 * p1))
TCAB_LAMBDA(MapExpMul, 2, (expf(p0) * p1))
TCAB_LAMBDA(MapSqMul, 2, ((p0 * p0) * p1))
TCAB_LAMBDA(MapAxpy, 2, ((c0 * p0) + (c1 * p1)))
TCAB_LAMBDA(MapScaleMul, 2, (((c0 * p0) + c1) * p1))
TCAB_LAMBDA(PostSelfRsqrt, 1, (p0 * rsqrtf(((p0 * c0) + c1))))
TCAB_LAMBDA(PostAddTanh, 1, (p0 + (c0 * tanhf(p0))))
TCAB_LAMBDA(PostScale, 1, (p0 * c0))

// map-only lambdas with an ahead-of-time kernel
TCAB_LAMBDA(MapScale, 1, (p0 * c0))
TCAB_LAMBDA(MapAffine, 1, ((p0 * c0) + c1))
TCAB_LAMBDA(MapAffineL, 1, ((c0 * p0) + c1))
TCAB_LAMBDA(MapRelu, 1, fmaxf(p0, c0))
TCAB_LAMBDA(MapExp, 1, expf(p0))
TCAB_LAMBDA(MapTanh, 1, tanhf(p0))
TCAB_LAMBDA(MapAdd2, 2, (p0 + p1))

// Partials of the multi-CTA split: at most this many per launch.
constexpr uint32_t kMaxSplitPartials = 262144;  // 1 MiB per (device, stream)

float* split_scratch(cudaStream_t stream);
int find_map_entry(const std::string& text, int n_in);

}  // namespace

// Middle-axis reductions with fewer column tiles than fill the SMs (less than half of the CTAs that can be resident,
// and fewer than four per SM) and a long k: how many CTAs share the k axis of a tile (1 = no split) -- as many as
// make the grid one resident wave, at least 256 k each, within the scratch.
// Pure arithmetic (no device query), so that it can be swept on a host without a GPU.
uint32_t plan_outer_splits(uint64_t tiles, uint64_t cells, uint32_t nk, uint64_t resident, int sms, int forced) {
  if (cells == 0 || cells > kMaxSplitPartials || tiles == 0) return 1;
  uint64_t want;
  if (forced > 0) {
    want = static_cast<uint64_t>(forced);  // forced by the tuning hook
  } else {
    // (measured bf16 [32, 4096, 1024]: 256 tiles on 148 SMs -- two CTAs per SM where eight fit -- 2.7 TB/s, with
    // the k axis cut so that the SMs are full 4.3+)
    if (tiles * 2 > resident || tiles >= 4 * static_cast<uint64_t>(sms)) return 1;
    want = resident / tiles;
    if (want > nk / 256) want = nk / 256;
  }
  if (want > kMaxSplitPartials / cells) want = kMaxSplitPartials / cells;
  if (want > nk) want = nk;
  return want < 2 ? 1 : static_cast<uint32_t>(want);
}

uint32_t choose_outer_splits(uint64_t tiles, uint64_t cells, uint32_t nk, uint64_t resident) {
  return plan_outer_splits(tiles, cells, nk, resident, sm_count(), tune(kReduceInner).p3);
}

// The ranges the launchers use: klen = ceil(nk / wanted), then as many ranges as cover [0, nk). Rounding
// klen up can leave fewer ranges than were wanted; a range beyond the last one would start past the end
// of the axis, so the count is recomputed from klen.
void plan_outer_ranges(uint32_t wanted, uint32_t nk, uint32_t* ranges, uint32_t* klen) {
  if (wanted < 2 || nk == 0) {
    *ranges = 1;
    *klen = nk;
    return;
  }
  *klen = (nk + wanted - 1) / wanted;
  *ranges = (nk + *klen - 1) / *klen;
}

// Rows folded by a warp each on a problem so small that all its CTAs are resident at once: 1024-thread CTAs.
// A launch costs by the CTA, and a small launch is bounded by exactly that cost (a [4096, 1024] input: 3.65 us
// per launch with 1024 CTAs of 128 threads, 3.33 us with 128 CTAs of 1024).
bool inner_wants_big_ctas(uint64_t rows) { return rows >= 64 && rows <= static_cast<uint64_t>(sm_count()) * 64; }

namespace {

struct Args {
  const float* const* ins;
  float* out;
  uint64_t outer;
  uint32_t nk;
  uint64_t inner;
  float init;
  Caps caps;
  cudaStream_t stream;
};

template <class Map, class Post, int COMBINE, int TPR, int V, int THREADS = tcabk::inner_cta_threads(TPR), int RAG = 0>
int launch_inner(const Args& a) {
  constexpr int NIN = Map::kIn;
  constexpr int GROUPS = THREADS / TPR;
  auto* fn = tcabk::chain_inner<Map, Post, COMBINE, NIN, TPR, V, 0, THREADS, 0, 0, RAG>;
  Ptrs<NIN> ptrs;
  for (int i = 0; i < NIN; ++i) ptrs.p[i] = a.ins[i];
  // one CTA per group of rows; the kernel's row loop only matters beyond 2^31 - 1 CTAs
  const uint64_t need = (a.outer + GROUPS - 1) / GROUPS;
  const uint64_t grid = need > 0x7fffffffull ? 0x7fffffffull : need;
  // Programmatic dependent launch: the grid may be scheduled while the previous kernel of the stream
  // drains (the kernel itself waits for it before touching memory), which hides most of the launch
  // gap between back-to-back small reductions. tune("reduce_inner", _, _, 2) switches it off.
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(grid));
  cfg.blockDim = dim3(THREADS);
  cfg.stream = a.stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = tune(kReduceInner).p2 == 2 ? 0 : 1;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, fn, ptrs, a.out, a.outer, a.nk, a.init, a.caps);
  count_launch();
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(TCAB_ERR_CUDA, "chain_inner: launch failed: %s", cudaGetErrorString(e));
  }
  return TCAB_OK;
}

// Rows of at most 16 vectors, a thread per row over a coalesced copy in shared memory: see chain_inner_rows32.
template <class Map, class Post, int COMBINE>
int launch_inner_rows32(const Args& a, uint32_t nvec, uint32_t warps) {
  constexpr int NIN = Map::kIn;
  auto* fn = tcabk::chain_inner_rows32<Map, Post, COMBINE, NIN>;
  Ptrs<NIN> ptrs;
  for (int i = 0; i < NIN; ++i) ptrs.p[i] = a.ins[i];
  const uint64_t rows_per_cta = static_cast<uint64_t>(warps) * 32;
  const uint64_t grid = (a.outer + rows_per_cta - 1) / rows_per_cta;
  if (grid > 0x7fffffffull) return fail(TCAB_ERR_TOO_LARGE, "chain_reduce: too many rows");
  const size_t smem = static_cast<size_t>(warps) * NIN * 32 * (nvec + 1) * 16;
  fn<<<static_cast<unsigned>(grid), 32 * warps, smem, a.stream>>>(ptrs, a.out, a.outer, nvec, a.init, a.caps);
  count_launch();
  return check_launch("chain_inner_rows32");
}

// Short rows that are not whole vectors, a thread per row over a copy of the rows as they lie: chain_inner_rows32e.
template <class Map, class Post, int COMBINE>
int launch_inner_rows32e(const Args& a, uint32_t warps) {
  constexpr int NIN = Map::kIn;
  auto* fn = tcabk::chain_inner_rows32e<Map, Post, COMBINE, NIN>;
  Ptrs<NIN> ptrs;
  for (int i = 0; i < NIN; ++i) ptrs.p[i] = a.ins[i];
  const uint64_t rows_per_cta = static_cast<uint64_t>(warps) * 32;
  const uint64_t grid = (a.outer + rows_per_cta - 1) / rows_per_cta;
  if (grid > 0x7fffffffull) return fail(TCAB_ERR_TOO_LARGE, "chain_reduce: too many rows");
  const size_t smem = static_cast<size_t>(warps) * NIN * 32 * a.nk * 4;
  fn<<<static_cast<unsigned>(grid), 32 * warps, smem, a.stream>>>(ptrs, a.out, a.outer, a.nk, a.init, a.caps);
  count_launch();
  return check_launch("chain_inner_rows32e");
}

// Short rows (at most 128 vectors): g lanes per row, VPL vectors per lane beyond 32, see chain_inner_flat.
template <class Map, class Post, int COMBINE, int VPL>
int launch_inner_flat_vpl(const Args& a, uint32_t nvec) {
  constexpr int NIN = Map::kIn;
  constexpr int UNROLL = 4;
  auto* fn = tcabk::chain_inner_flat<Map, Post, COMBINE, NIN, UNROLL, 0, VPL>;
  Ptrs<NIN> ptrs;
  for (int i = 0; i < NIN; ++i) ptrs.p[i] = a.ins[i];
  uint32_t g = 1;
  while (g < nvec && g < 32) g <<= 1;
  const uint64_t rows_per_cta = static_cast<uint64_t>(8) * UNROLL * (32 / g);
  const uint64_t grid = (a.outer + rows_per_cta - 1) / rows_per_cta;
  if (grid > 0x7fffffffull) return fail(TCAB_ERR_TOO_LARGE, "chain_reduce: too many rows");
  fn<<<static_cast<unsigned>(grid), 256, 0, a.stream>>>(ptrs, a.out, a.outer, nvec, g, a.init, a.caps);
  count_launch();
  return check_launch("chain_inner_flat");
}
template <class Map, class Post, int COMBINE>
int launch_inner_flat(const Args& a, uint32_t nvec) {
  if (nvec <= 32) return launch_inner_flat_vpl<Map, Post, COMBINE, 1>(a, nvec);
  return launch_inner_flat_vpl<Map, Post, COMBINE, 2>(a, nvec);
}

// The second launch of a split reduction: folds `splits` partials per output, several threads per output when there
// are many (finish_lanes).
template <class Post, int COMBINE>
int launch_finish(const float* scratch, float* out, uint32_t rows, uint32_t splits, float init, const Caps& caps,
                  cudaStream_t stream) {
  const uint32_t lanes = finish_lanes(splits);
  const uint64_t threads = static_cast<uint64_t>(rows) * lanes;
  tcabk::chain_split_finish<Post, COMBINE>
      <<<static_cast<unsigned>((threads + 127) / 128), 128, 0, stream>>>(scratch, out, rows, splits, init, caps, lanes);
  count_launch();
  return check_launch("chain_split_finish");
}

template <class Map, class Post, int COMBINE, int V>
int launch_outer_flat(const Args& a, uint32_t g) {
  constexpr int NIN = Map::kIn;
  // 4-byte loads need more of them in flight for the same bytes
  auto* fn = tcabk::chain_outer_flat<Map, Post, COMBINE, NIN, V == 4 ? 4 : 16, 0, 0, V>;
  Ptrs<NIN> ptrs;
  for (int i = 0; i < NIN; ++i) ptrs.p[i] = a.ins[i];
  const uint32_t nc = static_cast<uint32_t>(a.inner);
  const uint32_t tiles_per_b = (nc + 32 * V - 1) / (32 * V);
  const uint64_t work = a.outer * tiles_per_b;
  if (work > 0xffffffffull) return fail(TCAB_ERR_TOO_LARGE, "chain_reduce: too many column tiles");
  uint32_t klen = a.nk;
  uint32_t ksplit = outer_flat_ranges(a.outer, a.nk, nc, g, V == 4, sm_count(), kMaxSplitPartials, &klen);
  float* scratch = ksplit > 1 ? split_scratch(a.stream) : nullptr;
  if (scratch == nullptr) {
    ksplit = 1;
    klen = a.nk;
  }
  const uint64_t grid = ksplit > 1 ? work * ksplit : (work + 7) / 8;  // a CTA per range, or eight tiles per CTA
  fn<<<static_cast<unsigned>(grid), 256, 0, a.stream>>>(ptrs, a.out, static_cast<uint32_t>(a.outer), a.nk, nc, tiles_per_b, g,
                                                        a.init, a.caps, ksplit, klen, scratch);
  count_launch();
  int rc = check_launch("chain_outer_flat");
  if (rc != TCAB_OK || ksplit == 1) return rc;
  return launch_finish<Post, COMBINE>(scratch, a.out, static_cast<uint32_t>(a.outer * nc), ksplit, a.init, a.caps, a.stream);
}

template <class Map, class Post, int COMBINE, int V>
int launch_outer(const Args& a) {
  constexpr int NIN = Map::kIn;
  // 4-byte loads (rows that are not 16-byte multiples) need more of them in flight for the same bytes
  constexpr int KW = 8, UNROLL = V == 1 ? 8 : 4;
  auto* fn = tcabk::chain_outer<Map, Post, COMBINE, NIN, V, KW, UNROLL>;
  Ptrs<NIN> ptrs;
  for (int i = 0; i < NIN; ++i) ptrs.p[i] = a.ins[i];
  const uint32_t nc = static_cast<uint32_t>(a.inner);
  const uint32_t tiles_per_b = (nc + 32 * V - 1) / (32 * V);
  const uint64_t tiles = a.outer * tiles_per_b;
  if (tiles > 0xffffffffull) return fail(TCAB_ERR_TOO_LARGE, "chain_reduce: too many column tiles");
  const uint64_t cells = a.outer * nc;
  const int occ = occupancy(reinterpret_cast<const void*>(fn), 32 * KW, 0);
  uint32_t ksplit = choose_outer_splits(tiles, cells, a.nk, static_cast<uint64_t>(occ > 0 ? occ : 1) * sm_count());
  float* scratch = ksplit > 1 ? split_scratch(a.stream) : nullptr;
  if (scratch == nullptr) ksplit = 1;
  uint32_t klen = a.nk;
  plan_outer_ranges(ksplit, a.nk, &ksplit, &klen);  // no range starts at or past nk
  const uint64_t work = tiles * ksplit;
  const uint64_t grid = work > 0x7fffffffull ? 0x7fffffffull : work;  // one CTA per tile (and k range)
  fn<<<static_cast<unsigned>(grid), 32 * KW, 0, a.stream>>>(ptrs, a.out, static_cast<uint32_t>(a.outer), a.nk, nc,
                                                          tiles_per_b, a.init, a.caps, ksplit, klen, scratch);
  count_launch();
  int rc = check_launch("chain_outer");
  if (rc != TCAB_OK || ksplit == 1) return rc;
  return launch_finish<Post, COMBINE>(scratch, a.out, static_cast<uint32_t>(cells), ksplit, a.init, a.caps, a.stream);
}

// How many CTAs share one row: 1 = no split. A split pays off when there are fewer rows than SMs and
// the rows are long; the number of partials is bounded by the scratch buffer.
uint32_t choose_splits(uint64_t rows, uint32_t nvec) {
  const Tune& tn = tune(kReduceInner);
  if (rows == 0 || rows > kMaxSplitPartials) return 1;
  uint64_t s;
  if (tn.p1 > 0) {
    s = static_cast<uint64_t>(tn.p1);
  } else {
    if (rows >= static_cast<uint64_t>(sm_count()) || nvec < 4096) return 1;
    s = (4ull * sm_count() + rows - 1) / rows;           // about four CTAs per SM in total
    const uint64_t by_len = (nvec + 1023) / 1024;         // at least 1024 vectors per CTA
    if (s > by_len) s = by_len;
  }
  if (s > nvec) s = nvec;
  if (s * rows > kMaxSplitPartials) s = kMaxSplitPartials / rows;
  return s < 1 ? 1u : static_cast<uint32_t>(s);
}

template <class Map, class Post, int COMBINE, int V>
int launch_split(const Args& a, float* scratch, uint32_t nvec, uint32_t splits) {
  constexpr int NIN = Map::kIn;
  Ptrs<NIN> ptrs;
  for (int i = 0; i < NIN; ++i) ptrs.p[i] = a.ins[i];
  const uint32_t rows = static_cast<uint32_t>(a.outer);
  const uint32_t vec_per_split = (nvec + splits - 1) / splits;
  tcabk::chain_inner_split<Map, COMBINE, NIN, V>
      <<<rows * splits, 256, 0, a.stream>>>(ptrs, scratch, a.nk, splits, vec_per_split, a.caps);
  count_launch();
  int rc = check_launch("chain_inner_split");
  if (rc != TCAB_OK) return rc;
  return launch_finish<Post, COMBINE>(scratch, a.out, rows, splits, a.init, a.caps, a.stream);
}

template <class Map, class Post, int COMBINE>
int launch_chain(const Args& a) {
  constexpr int NIN = Map::kIn;
  bool al = true;
  for (int i = 0; i < NIN; ++i) al = al && aligned16(a.ins[i]);
  if (a.inner == 1) {
    const bool vec = al && (a.nk % 4 == 0);
    const uint32_t nvec = vec ? a.nk / 4 : a.nk;
    const uint32_t splits = choose_splits(a.outer, nvec);
    if (splits > 1) {
      float* scratch = split_scratch(a.stream);  // null only if the allocation failed: no split then
      if (scratch != nullptr)
        return vec ? launch_split<Map, Post, COMBINE, 4>(a, scratch, nvec, splits)
                   : launch_split<Map, Post, COMBINE, 1>(a, scratch, nvec, splits);
    }
    // short rows with enough of them: lanes along the row, consecutive rows in a warp (tune p0 keeps chain_inner)
    // up to 16 vectors a thread still folds its row in the reference's ascending order, over a coalesced copy
    // (a row of one vector needs no copy: a lane folds its own vector in order)
    if (vec && nvec >= 2 && nvec <= 16 && a.outer >= 1024 && tune(kReduceInner).p0 <= 0 && rows32_warps(nvec, NIN) >= 2)
      return launch_inner_rows32<Map, Post, COMBINE>(a, nvec, rows32_warps(nvec, NIN));
    // (measured: up to 32 vectors, and 49 ... 64 with two vectors per lane; other lengths up to 128 were no faster)
    if (vec && nvec >= 1 && (nvec <= 32 || (nvec > 48 && nvec <= 64)) && a.outer >= 1024 && tune(kReduceInner).p0 <= 0)
      return launch_inner_flat<Map, Post, COMBINE>(a, nvec);
    // short rows: one thread folds a row sequentially, which is the reference's SeqReducer order exactly
    // measured: a warp per row for mid-length rows, a CTA per row for long ones (8192 columns: 4.6 -> 7.1 TB/s)
    // (a CTA per row from 640 vectors, from 384 with two or more operands: 3072 columns 6.4 -> 7.1 TB/s, 4092 5.1 -> 6.8,
    //  two operands at 1536 columns 6.9 -> 7.4)
    // rows that are not whole vectors on aligned operands: up to 64 elements a thread per row over a copy of the rows
    // as they lie; longer rows with 16-byte loads between their ragged ends (tune p0 keeps the 4-byte kernels)
    if (al && !vec && tune(kReduceInner).p0 <= 0) {
      if (a.nk <= 64 && a.outer >= 1024 && rows32e_warps(a.nk, NIN) >= 1)
        return launch_inner_rows32e<Map, Post, COMBINE>(a, rows32e_warps(a.nk, NIN));
      if (a.nk > 64)  // the thresholds of whole-vector rows
        return a.nk / 4 <= 64                            ? launch_inner<Map, Post, COMBINE, 4, 4, 128, 1>(a)
               : a.nk / 4 < inner_cta_per_row_from(NIN) ? launch_inner<Map, Post, COMBINE, 32, 4, 128, 1>(a)
                                                        : launch_inner<Map, Post, COMBINE, 256, 4, 256, 1>(a);
    }
    int tpr = nvec <= 16 ? 1 : nvec <= 64 ? 4 : nvec < (vec ? inner_cta_per_row_from(NIN) : 1024u) ? 32 : 256;
    const Tune& tn = tune(kReduceInner);
    if (tn.p0 == 1 || tn.p0 == 4 || tn.p0 == 32 || tn.p0 == 256) tpr = tn.p0;
    if (vec) {
      switch (tpr) {
        case 1: return launch_inner<Map, Post, COMBINE, 1, 4>(a);
        case 4: return launch_inner<Map, Post, COMBINE, 4, 4>(a);
        case 32:
          if (inner_wants_big_ctas(a.outer) && tn.p2 != 3) return launch_inner<Map, Post, COMBINE, 32, 4, 1024>(a);
          return launch_inner<Map, Post, COMBINE, 32, 4>(a);
        default: return launch_inner<Map, Post, COMBINE, 256, 4>(a);
      }
    }
    switch (tpr) {
      case 1: return launch_inner<Map, Post, COMBINE, 1, 1>(a);
      case 4: return launch_inner<Map, Post, COMBINE, 4, 1>(a);
      case 32: return launch_inner<Map, Post, COMBINE, 32, 1>(a);
      default: return launch_inner<Map, Post, COMBINE, 256, 1>(a);
    }
  }
  if (a.inner > 0xffffffffull) return fail(TCAB_ERR_TOO_LARGE, "chain_reduce: inner extent beyond 2^32");
  const bool vec = al && (a.inner % 4 == 0);
  // narrow rows and short reduced axes: a warp per (b, column tile) (outer_flat_groups has the rule and the
  // measurements). tune("reduce_inner", _, _, _, p3 = 1) keeps chain_outer, p0 = 32 takes the warps whatever the shape.
  if (tune(kReduceInner).p3 <= 0) {
    const uint32_t nc = static_cast<uint32_t>(a.inner);
    const uint32_t g = tune(kReduceInner).p0 == 32 ? outer_flat_width(nc, vec) : outer_flat_groups(a.outer, a.nk, nc, sm_count(), vec);
    if (g != 0) return vec ? launch_outer_flat<Map, Post, COMBINE, 4>(a, g) : launch_outer_flat<Map, Post, COMBINE, 1>(a, g);
  }
  return vec ? launch_outer<Map, Post, COMBINE, 4>(a) : launch_outer<Map, Post, COMBINE, 1>(a);
}

// Several problems of one shape in one launch (chain_inner_batched): a warp per row below 1024 vectors, a CTA per
// row from there.
struct BatchArgs {
  const float* const* ins;   // [nprob][n_in]
  float* const* outs;        // [nprob]
  uint32_t nprob;
  uint32_t rows, nk;
  float init;
  Caps caps;
  cudaStream_t stream;
};

template <class Map, class Post, int COMBINE>
int launch_batched(const BatchArgs& a) {
  constexpr int NIN = Map::kIn;
  tcabk::BatchPtrs<NIN> ptrs = {};
  bool al = true;
  for (uint32_t b = 0; b < a.nprob; ++b) {
    for (int i = 0; i < NIN; ++i) {
      ptrs.in[b][i] = a.ins[b * NIN + i];
      al = al && aligned16(ptrs.in[b][i]);
    }
    ptrs.out[b] = a.outs[b];
  }
  const bool vec = al && (a.nk % 4 == 0);
  const uint32_t nvec = vec ? a.nk / 4 : a.nk;
  const bool cta_per_row = nvec >= 1024;
  const uint64_t total = static_cast<uint64_t>(a.nprob) * a.rows;
  const uint64_t need = cta_per_row ? total : (total + 7) / 8;
  const unsigned grid = static_cast<unsigned>(need > 0x7fffffffull ? 0x7fffffffull : need);
  void (*fn)(tcabk::BatchPtrs<NIN>, uint32_t, uint32_t, uint32_t, float, Caps) =
      vec ? (cta_per_row ? tcabk::chain_inner_batched<Map, Post, COMBINE, NIN, 256, 4>
                         : tcabk::chain_inner_batched<Map, Post, COMBINE, NIN, 32, 4>)
          : (cta_per_row ? tcabk::chain_inner_batched<Map, Post, COMBINE, NIN, 256, 1>
                         : tcabk::chain_inner_batched<Map, Post, COMBINE, NIN, 32, 1>);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(256);
  cfg.stream = a.stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = tune(kReduceInner).p2 == 2 ? 0 : 1;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, fn, ptrs, a.nprob, a.rows, a.nk, a.init, a.caps);
  count_launch();
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(TCAB_ERR_CUDA, "chain_inner_batched: launch failed: %s", cudaGetErrorString(e));
  }
  return TCAB_OK;
}

// The split path on a scratch buffer the caller of this function provides (used by the entry point
// that allocates nothing): always two launches, whatever the shape.
template <class Map, class Post, int COMBINE>
int launch_split_on(const Args& a, float* scratch, uint32_t splits) {
  constexpr int NIN = Map::kIn;
  bool al = true;
  for (int i = 0; i < NIN; ++i) al = al && aligned16(a.ins[i]);
  const bool vec = al && (a.nk % 4 == 0);
  const uint32_t nvec = vec ? a.nk / 4 : a.nk;
  if (splits > nvec) splits = nvec > 0 ? nvec : 1;
  return vec ? launch_split<Map, Post, COMBINE, 4>(a, scratch, nvec, splits)
             : launch_split<Map, Post, COMBINE, 1>(a, scratch, nvec, splits);
}

struct Entry {
  const char* map;
  const char* post;  // "" = the reduction is stored as it is
  int combine;
  int n_in;
  int (*launch)(const Args&);
  int (*launch_noalloc)(const Args&, float* scratch, uint32_t splits);  // split path on caller-free scratch
  int (*launch_batched)(const BatchArgs&);                              // several problems of one shape in one launch
};

#define TCAB_ENTRY(MAP, POST, COMBINE)                                            \
  { MAP::text(), POST::text(), COMBINE, MAP::kIn, &launch_chain<MAP, POST, COMBINE>, \
    &launch_split_on<MAP, POST, COMBINE>, &launch_batched<MAP, POST, COMBINE> }
#define TCAB_ENTRY_NOPOST(MAP, COMBINE)                                                  \
  { MAP::text(), "", COMBINE, MAP::kIn, &launch_chain<MAP, tcabk::PostNone, COMBINE>,    \
    &launch_split_on<MAP, tcabk::PostNone, COMBINE>, &launch_batched<MAP, tcabk::PostNone, COMBINE> }

const Entry kTable[] = {
    TCAB_ENTRY_NOPOST(MapIdent, 0),    TCAB_ENTRY_NOPOST(MapIdent, 1),    TCAB_ENTRY_NOPOST(MapIdent, 2),
    TCAB_ENTRY_NOPOST(MapAffineSq, 0), TCAB_ENTRY_NOPOST(MapMul2, 0),     TCAB_ENTRY_NOPOST(MapExpMul, 0),
    TCAB_ENTRY_NOPOST(MapScaleMul, 0), TCAB_ENTRY(MapSqMul, PostSelfRsqrt, 0),
    TCAB_ENTRY(MapAxpy, PostAddTanh, 0), TCAB_ENTRY(MapMul2, PostScale, 0),
};

// Scratch for the partials of the split path: kMaxSplitPartials floats per (device, stream).
float* split_scratch(cudaStream_t stream) {
  return static_cast<float*>(stream_scratch(kScratchChainSplit, stream, kMaxSplitPartials * sizeof(float), false));
}

// ---- map-only chains ----------------------------------------------------------------------------------
struct MapArgs {
  const void* const* ins;
  void* out;
  uint64_t n;
  Caps caps;
  cudaStream_t stream;
};

template <class Map>
int launch_map_aot(const MapArgs& a) {
  constexpr int NIN = Map::kIn;
  Ptrs<NIN> ptrs;
  bool al = aligned16(a.out);
  for (int i = 0; i < NIN; ++i) {
    ptrs.p[i] = static_cast<const float*>(a.ins[i]);
    al = al && aligned16(a.ins[i]);
  }
  if (al) {
    const uint64_t threads = a.n / 8 + 1;  // one thread per group of eight, one more for the ragged end
    tcabk::chain_map<Map, NIN, 0, false, 8>
        <<<static_cast<unsigned>((threads + 255) / 256), 256, 0, a.stream>>>(ptrs, a.out, a.n, a.caps, 0u);
  } else {
    tcabk::chain_map<Map, NIN, 0, false, 1>
        <<<static_cast<unsigned>((a.n + 255) / 256), 256, 0, a.stream>>>(ptrs, a.out, a.n, a.caps, 0u);
  }
  count_launch();
  return check_launch("chain_map");
}

struct MapEntry {
  const char* map;
  int n_in;
  int (*launch)(const MapArgs&);
};
#define TCAB_MAP_ENTRY(MAP) { MAP::text(), MAP::kIn, &launch_map_aot<MAP> }
const MapEntry kMapTable[] = {
    TCAB_MAP_ENTRY(MapIdent),  TCAB_MAP_ENTRY(MapAffineSq), TCAB_MAP_ENTRY(MapScale), TCAB_MAP_ENTRY(MapAffine),
    TCAB_MAP_ENTRY(MapAffineL), TCAB_MAP_ENTRY(MapRelu),    TCAB_MAP_ENTRY(MapExp),   TCAB_MAP_ENTRY(MapTanh),
    TCAB_MAP_ENTRY(MapAdd2),   TCAB_MAP_ENTRY(MapMul2),
};

int find_map_entry(const std::string& text, int n_in) {
  for (size_t i = 0; i < sizeof(kMapTable) / sizeof(kMapTable[0]); ++i)
    if (kMapTable[i].n_in == n_in && text == kMapTable[i].map) return static_cast<int>(i);
  return -1;
}

int combine_id(const std::string& text) {
  if (text == "(p0 + p1)" || text == "(p1 + p0)") return 0;
  if (text == "fmaxf(p0, p1)" || text == "fmaxf(p1, p0)") return 1;
  if (text == "fminf(p0, p1)" || text == "fminf(p1, p0)") return 2;
  return -1;
}

}  // namespace

namespace {
int prepare_chain_uncached(const tcab_chain* chain, uint32_t n_ins, PreparedChain* pc, char kind, const int* in_types,
                           int out_type, int rb_mask, int cb_mask, int cell_mask);
}  // namespace

// A host calls with the same few lambdas over and over: the last prepared chains of a thread are kept, keyed by
// everything that went into them (the texts, the capture values, the operand types, the indexing masks), so that a
// repeated call skips parsing and canonicalising three expressions (measured: a third of a small launch's host time).
int prepare_chain(const tcab_chain* chain, uint32_t n_ins, PreparedChain* pc, char kind, const int* in_types, int out_type,
                  int rb_mask, int cb_mask, int cell_mask) {
  if (chain == nullptr || chain->map_expr == nullptr || chain->n_captures > TCAB_MAX_CAPTURES || n_ins > TCAB_MAX_INPUTS)
    return prepare_chain_uncached(chain, n_ins, pc, kind, in_types, out_type, rb_mask, cb_mask, cell_mask);
  thread_local std::vector<std::pair<std::string, PreparedChain>> cache;
  std::string key;
  key.reserve(160);
  key.push_back(kind);
  key.push_back(static_cast<char>('0' + n_ins));
  for (uint32_t i = 0; i < n_ins; ++i) key.push_back(static_cast<char>('0' + (in_types != nullptr ? in_types[i] : 0)));
  const int small[4] = {out_type, rb_mask, cb_mask, cell_mask};
  key.append(reinterpret_cast<const char*>(small), sizeof(small));
  key.append(reinterpret_cast<const char*>(&chain->init), sizeof(float));
  key.append(reinterpret_cast<const char*>(chain->captures), sizeof(float) * chain->n_captures);
  key.push_back('\x1f');
  key.append(chain->map_expr);
  key.push_back('\x1f');
  if (chain->combine_expr != nullptr) key.append(chain->combine_expr);
  key.push_back('\x1f');
  if (chain->post_expr != nullptr) key.append(chain->post_expr);
  for (const auto& e : cache)
    if (e.first == key) {
      *pc = e.second;
      return TCAB_OK;
    }
  const int rc = prepare_chain_uncached(chain, n_ins, pc, kind, in_types, out_type, rb_mask, cb_mask, cell_mask);
  if (rc == TCAB_OK) {
    if (cache.size() >= 16) cache.erase(cache.begin());
    cache.emplace_back(std::move(key), *pc);
  }
  return rc;
}

namespace {
int prepare_chain_uncached(const tcab_chain* chain, uint32_t n_ins, PreparedChain* pc, char kind, const int* in_types,
                           int out_type, int rb_mask, int cb_mask, int cell_mask) {
  const char* op = kind == 'M' ? "map" : kind == 'C' ? "chain_contract" : "chain_reduce";
  std::vector<float> user(chain->captures, chain->captures + chain->n_captures);
  CanonExpr map, comb, post;
  std::string err;
  ElemT types[TCAB_MAX_INPUTS] = {};  // kF32 == 0
  bool all_f32 = true;
  for (uint32_t i = 0; i < n_ins && in_types != nullptr; ++i) {
    types[i] = static_cast<ElemT>(in_types[i]);
    all_f32 = all_f32 && in_types[i] == TCAB_F32;
  }
  if (!canonicalize(chain->map_expr, static_cast<int>(n_ins), types, user, &map, &err))
    return fail(TCAB_ERR_INVALID_ARG, "%s: map_expr: %s", op, err.c_str());
  if (map.n_operands != static_cast<int>(n_ins))
    return fail(TCAB_ERR_INVALID_ARG, "%s: map_expr uses %d operands, %u given", op, map.n_operands, n_ins);
  if (map.captures.size() > 8) return fail(TCAB_ERR_UNSUPPORTED, "%s: more than 8 distinct constants in one lambda", op);
  for (int i = 0; i < 16; ++i) pc->caps[i] = 0.0f;
  for (size_t i = 0; i < map.captures.size(); ++i) pc->caps[i] = map.captures[i];
  pc->init = chain->init;
  pc->entry = -1;
  JitSpec& sp = pc->spec;
  sp = JitSpec();
  sp.kind = kind;
  sp.n_in = static_cast<int>(n_ins);
  for (uint32_t i = 0; i < n_ins; ++i) sp.in_types[i] = static_cast<int>(types[i]);
  sp.out_type = out_type;
  sp.rb_mask = rb_mask;
  sp.cb_mask = cb_mask;
  sp.cell_mask = cell_mask;
  if ((rb_mask | cb_mask | cell_mask) != 0) all_f32 = false;  // broadcast operands: compiled at run time only
  sp.map_text = map.text;
  if (kind == 'M') {
    // a map-only chain stores the lambda's value as it is: its type is the output's element type, no conversion
    // is implied (casts are always explicit, internal/ir/types.go:60-62)
    if (static_cast<int>(map.type) != out_type)
      return fail(TCAB_ERR_DTYPE, "map: the lambda yields %s but out holds %s; convert explicitly (static_cast)",
                  elem_name(map.type), elem_name(static_cast<ElemT>(out_type)));
    if (all_f32 && out_type == TCAB_F32) pc->entry = find_map_entry(map.text, static_cast<int>(n_ins));
    if (pc->entry < 0) pc->entry = kJitEntry;
    return TCAB_OK;
  }
  // reductions and contractions fold f32 values (homogeneous reducers: pkg/chain.go:229-264)
  if (map.type != kF32)
    return fail(TCAB_ERR_DTYPE, "%s: the map lambda yields %s; this class folds f32 values, convert explicitly", op,
                elem_name(map.type));
  if (!canonicalize(chain->combine_expr, 2, nullptr, {}, &comb, &err))
    return fail(TCAB_ERR_INVALID_ARG, "%s: combine_expr: %s", op, err.c_str());
  const bool has_post = chain->post_expr != nullptr && chain->post_expr[0] != '\0';
  if (has_post && !canonicalize(chain->post_expr, 1, nullptr, user, &post, &err))
    return fail(TCAB_ERR_INVALID_ARG, "%s: post_expr: %s", op, err.c_str());
  if (has_post && post.type != kF32)
    return fail(TCAB_ERR_DTYPE, "%s: the piped map yields %s; out holds f32", op, elem_name(post.type));
  const int cid = combine_id(comb.text);
  if (cid < 0) return fail(TCAB_ERR_UNSUPPORTED, "%s: combiner '%s' is not sum/fmaxf/fminf", op, comb.text.c_str());
  if (post.captures.size() > 8) return fail(TCAB_ERR_UNSUPPORTED, "%s: more than 8 distinct constants in one lambda", op);
  for (size_t i = 0; i < post.captures.size(); ++i) pc->caps[8 + i] = post.captures[i];
  sp.combine = cid;
  sp.post_text = has_post ? post.text : std::string();
  if (all_f32) {
    for (size_t i = 0; i < sizeof(kTable) / sizeof(kTable[0]); ++i) {
      const Entry& e = kTable[i];
      if (e.combine == cid && e.n_in == static_cast<int>(n_ins) && map.text == e.map && sp.post_text == e.post) {
        pc->entry = static_cast<int>(i);
        return TCAB_OK;
      }
    }
  }
  // no ahead-of-time instance: compiled at run time on the first launch (chain_jit.cu)
  pc->entry = kJitEntry;
  return TCAB_OK;
}
}  // namespace

int launch_chain_reduce(const PreparedChain& pc, const float* const* ins, uint64_t outer, uint32_t nk,
                        uint64_t inner, float* out, cudaStream_t s) {
  if (outer == 0 || inner == 0) return TCAB_OK;
  if (pc.entry == kJitEntry) {
    void* h = nullptr;
    const int rc = jit_prepare(pc.spec, &h);
    if (rc != TCAB_OK) return rc;
    uint32_t splits = 1;
    float* scratch = nullptr;
    if (inner == 1) {
      bool al = true;
      for (int i = 0; i < pc.spec.n_in; ++i) al = al && aligned16(ins[i]);
      splits = (pc.spec.rb_mask | pc.spec.cb_mask) ? 1 : choose_splits(outer, (al && nk % 4 == 0) ? nk / 4 : nk);
      if (splits > 1) scratch = split_scratch(s);
    } else if (outer * ((inner + 31) / 32) < 16ull * static_cast<uint64_t>(sm_count()) && nk >= 512) {
      scratch = split_scratch(s);  // a middle-axis reduction that may split k over CTAs (decided at launch)
    }
    return jit_launch(h, ins, outer, nk, inner, pc.init, pc.caps, out, scratch, splits, s);
  }
  Args a{ins, out, outer, nk, inner, pc.init, {}, s};
  for (int i = 0; i < 16; ++i) a.caps.c[i] = pc.caps[i];
  return kTable[pc.entry].launch(a);
}

int launch_chain_reduce_batched(const PreparedChain& pc, const float* const* ins, float* const* outs, uint32_t nprob,
                                uint32_t rows, uint32_t nk, cudaStream_t s) {
  if (nprob == 0 || rows == 0) return TCAB_OK;
  if (pc.entry == kJitEntry) {
    JitSpec sp = pc.spec;
    sp.kind = 'B';
    void* h = nullptr;
    const int rc = jit_prepare(sp, &h);
    if (rc != TCAB_OK) return rc;
    return jit_launch_batched(h, ins, outs, nprob, rows, nk, pc.init, pc.caps, s);
  }
  BatchArgs a{ins, outs, nprob, rows, nk, pc.init, {}, s};
  for (int i = 0; i < 16; ++i) a.caps.c[i] = pc.caps[i];
  return kTable[pc.entry].launch_batched(a);
}

int launch_chain_map(const PreparedChain& pc, const void* const* ins, void* out, uint64_t n, uint32_t cols, cudaStream_t s) {
  if (n == 0) return TCAB_OK;
  if (n / 8 / 256 >= 0x7fffffffull) return fail(TCAB_ERR_TOO_LARGE, "map: too many elements for one launch");
  if (pc.entry == kJitEntry) {
    void* h = nullptr;
    const int rc = jit_prepare(pc.spec, &h);
    if (rc != TCAB_OK) return rc;
    return jit_launch_map(h, ins, out, n, cols, pc.caps, s);
  }
  MapArgs a{ins, out, n, {}, s};
  for (int i = 0; i < 16; ++i) a.caps.c[i] = pc.caps[i];
  return kMapTable[pc.entry].launch(a);
}

// The chain as the run-time compiler sees it when it is launched as a contraction: a chain found in the
// reduce table carries that table's lambdas.
JitSpec contract_spec(const PreparedChain& pc) {
  JitSpec sp = pc.spec;
  sp.kind = 'C';
  sp.n_in = 2;
  return sp;
}

bool contract_is_aot(const PreparedChain& pc) {
  return pc.entry >= 0 && kTable[pc.entry].combine == 0 && std::string(kTable[pc.entry].map) == MapMul2::text() &&
         (std::string(kTable[pc.entry].post).empty() || std::string(kTable[pc.entry].post) == PostScale::text());
}

// Compiles and loads the kernels of a chain that has no ahead-of-time instance (nothing to do otherwise).
int warm_chain(const PreparedChain& pc) {
  void* h = nullptr;
  if (pc.spec.kind == 'C') return contract_is_aot(pc) ? TCAB_OK : jit_prepare(contract_spec(pc), &h);
  if (pc.entry != kJitEntry) return TCAB_OK;
  return jit_prepare(pc.spec, &h);
}

// ---------------------------------------------------------------------------
// fp32 contraction chains
// ---------------------------------------------------------------------------
bool contract_big_tiles(uint32_t m, uint32_t n);

namespace {

template <class Map, class Post, int COMBINE>
int launch_contract_aot(const float* lhs, const float* rhs, float* out, uint32_t m, uint32_t n, uint32_t k,
                        int rhs_nk, float init, const Caps& caps, cudaStream_t s) {
  if (contract_big_tiles(m, n)) {
    const dim3 grid((n + 127) / 128, (m + 127) / 128);
    if (rhs_nk)
      tcabk::chain_contract<Map, Post, COMBINE, 1, 8><<<grid, 256, 0, s>>>(lhs, rhs, out, m, n, k, init, caps);
    else
      tcabk::chain_contract<Map, Post, COMBINE, 0, 8><<<grid, 256, 0, s>>>(lhs, rhs, out, m, n, k, init, caps);
  } else {
    const dim3 grid((n + 63) / 64, (m + 63) / 64);
    if (rhs_nk)
      tcabk::chain_contract<Map, Post, COMBINE, 1, 4><<<grid, 256, 0, s>>>(lhs, rhs, out, m, n, k, init, caps);
    else
      tcabk::chain_contract<Map, Post, COMBINE, 0, 4><<<grid, 256, 0, s>>>(lhs, rhs, out, m, n, k, init, caps);
  }
  count_launch();
  return check_launch("chain_contract");
}

}  // namespace

// 128x128 tiles once they fill the GPU (two CTAs per SM are resident), 64x64 tiles below that.
bool contract_big_tiles(uint32_t m, uint32_t n) {
  const Tune& tn = tune(kGemm);
  if (tn.p2 == 4) return false;
  if (tn.p2 == 8) return true;
  const uint64_t tiles = static_cast<uint64_t>((m + 127) / 128) * ((n + 127) / 128);
  return tiles >= static_cast<uint64_t>(sm_count());
}

int launch_chain_contract(const PreparedChain& pc, const float* lhs, const float* rhs, int rhs_nk, float* out,
                          uint32_t m, uint32_t n, uint32_t k, cudaStream_t s) {
  if (m == 0 || n == 0) return TCAB_OK;
  if ((n + 63) / 64 > 65535u * 64u || (m + 63) / 64 > 65535u)
    return fail(TCAB_ERR_TOO_LARGE, "chain_contract: more than 65535 row tiles");
  Caps caps;
  for (int i = 0; i < 16; ++i) caps.c[i] = pc.caps[i];
  // bf16 x bf16 with the plain product, a sum reducer and init 0, stored as it is or scaled: that is a tensor-core
  // contraction with fp32 accumulation (products of bf16 values are exact in fp32, so only the order of the sum
  // differs from the scalar kernel). Needs 16-byte rows and pointers; tune("gemm", _, _, 64) keeps the scalar kernel.
  if (pc.spec.in_types[0] == TCAB_BF16 && pc.spec.in_types[1] == TCAB_BF16 && pc.spec.combine == 0 &&
      pc.init == 0.0f && pc.spec.map_text == "(static_cast<float>(p0) * static_cast<float>(p1))" &&
      (pc.spec.post_text.empty() || pc.spec.post_text == "(p0 * c0)" || pc.spec.post_text == "(c0 * p0)") &&
      k % 8 == 0 && n % 4 == 0 && (rhs_nk || n % 8 == 0) && ((reinterpret_cast<uintptr_t>(lhs) | reinterpret_cast<uintptr_t>(rhs) |
                                                              reinterpret_cast<uintptr_t>(out)) & 15u) == 0 &&
      tune(kGemm).p2 != 64) {
    const float alpha = pc.spec.post_text.empty() ? 1.0f : pc.caps[8];  // the piped map's first constant
    return launch_contract_bf16_tc(reinterpret_cast<const __nv_bfloat16*>(lhs), reinterpret_cast<const __nv_bfloat16*>(rhs), rhs_nk,
                                   alpha, out, m, n, k, s);
  }
  // ahead-of-time: the plain product with a sum reducer, stored as it is or scaled
  if (pc.entry >= 0 && kTable[pc.entry].combine == 0 && std::string(kTable[pc.entry].map) == MapMul2::text()) {
    const std::string post = kTable[pc.entry].post;
    // large fp32 problems: three bf16 pieces per operand on the tensor cores (tune("gemm", _, _, 64) keeps the scalar
    // kernel; so do small problems, whose outputs then keep the reference's ascending order over k)
    if (pc.init == 0.0f && (post.empty() || post == PostScale::text()) && tune(kGemm).p2 != 64) {
      const int rc = launch_contract_f32_split3(lhs, rhs, rhs_nk, post.empty() ? 1.0f : pc.caps[8], out, m, n, k, s);
      if (rc != TCAB_ERR_UNSUPPORTED) return rc;
    }
    if (post.empty())
      return launch_contract_aot<MapMul2, tcabk::PostNone, 0>(lhs, rhs, out, m, n, k, rhs_nk, pc.init, caps, s);
    if (post == PostScale::text())
      return launch_contract_aot<MapMul2, PostScale, 0>(lhs, rhs, out, m, n, k, rhs_nk, pc.init, caps, s);
  }
  void* h = nullptr;
  const int rc = jit_prepare(contract_spec(pc), &h);
  if (rc != TCAB_OK) return rc;
  return jit_launch_contract(h, lhs, rhs, rhs_nk, out, m, n, k, pc.init, pc.caps, s);
}

// ---------------------------------------------------------------------------
// The entry point that allocates nothing
// ---------------------------------------------------------------------------
// Scratch for the split path when the caller cannot let the library allocate: a fixed array in
// device memory, part of the library image. Every GPU that loads the library holds these 16 KiB
// until the process exits. Every call on a device shares the array.
constexpr uint32_t kNoAllocMaxPartials = TCAB_NOALLOC_MAX_ROWS;
static __device__ __align__(256) float g_noalloc_scratch[kNoAllocMaxPartials];

namespace {

// In host code `g_noalloc_scratch` names a host-side shadow of the array, not its device address;
// a kernel handed that name would read and write the wrong memory. The device address comes from
// cudaGetSymbolAddress, asked once per device with that device current.
constexpr int kMaxDevices = 64;
float* g_noalloc_ptr[kMaxDevices] = {};
std::mutex g_noalloc_mu;

int noalloc_scratch(float** out) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) {
    cudaGetLastError();
    return fail(TCAB_ERR_CUDA, "chain_reduce_noalloc: no current CUDA device");
  }
  if (dev < 0 || dev >= kMaxDevices)
    return fail(TCAB_ERR_UNSUPPORTED, "chain_reduce_noalloc: device ordinal %d beyond %d", dev, kMaxDevices - 1);
  std::lock_guard<std::mutex> lk(g_noalloc_mu);
  if (g_noalloc_ptr[dev] == nullptr) {
    void* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess || p == nullptr) {
      cudaGetLastError();
      return fail(TCAB_ERR_CUDA, "chain_reduce_noalloc: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
    }
    g_noalloc_ptr[dev] = static_cast<float*>(p);
  }
  *out = g_noalloc_ptr[dev];
  return TCAB_OK;
}

}  // namespace

int launch_chain_reduce_noalloc(const PreparedChain& pc, const float* const* ins, uint64_t rows, uint32_t nk,
                                float* out, cudaStream_t s) {
  if (rows > kNoAllocMaxPartials)
    return fail(TCAB_ERR_TOO_LARGE,
                "chain_reduce_noalloc: %llu rows, but the fixed scratch array holds %u partial results "
                "(one per row at least); use tcab_chain_reduce for larger problems",
                static_cast<unsigned long long>(rows), kNoAllocMaxPartials);
  if (rows == 0) return TCAB_OK;
  if ((pc.spec.rb_mask | pc.spec.cb_mask) != 0)
    return fail(TCAB_ERR_UNSUPPORTED, "chain_reduce_noalloc: operands with broadcast extents are not taken by the split kernels");
  float* scratch = nullptr;
  const int rc = noalloc_scratch(&scratch);
  if (rc != TCAB_OK) return rc;
  // As many CTAs per row as the array has room for, up to about four CTAs per SM in total and at
  // least 1024 vectors per CTA. Every partial that pass 2 reads is written by pass 1 of the same call
  // (a CTA with an empty range writes the combiner's identity), so nothing in the array has to be
  // cleared between calls.
  uint64_t splits = (4ull * sm_count() + rows - 1) / rows;
  const uint64_t by_len = (static_cast<uint64_t>(nk) / 4 + 1023) / 1024;
  if (splits > by_len) splits = by_len;
  if (splits * rows > kNoAllocMaxPartials) splits = kNoAllocMaxPartials / rows;
  if (splits < 1) splits = 1;
  if (pc.entry == kJitEntry) {
    // Never compiled here: compiling loads a code image onto the device, which allocates device memory.
    void* h = nullptr;
    const int jrc = jit_prepare(pc.spec, &h, false);
    if (jrc != TCAB_OK)
      return fail(TCAB_ERR_UNSUPPORTED,
                  "chain_reduce_noalloc: the lambda '%s' has no ahead-of-time kernel and has not been compiled in this "
                  "process yet; call tcab_chain_prepare (or tcab_chain_reduce) with it once, outside any capture",
                  pc.spec.map_text.c_str());
    // the split kernels always: splits may be 1, the partials still pass through the fixed array
    return jit_launch(h, ins, rows, nk, 1, pc.init, pc.caps, out, scratch, static_cast<uint32_t>(splits) | 0x80000000u, s);
  }
  Args a{ins, out, rows, nk, 1, pc.init, {}, s};
  for (int i = 0; i < 16; ++i) a.caps.c[i] = pc.caps[i];
  return kTable[pc.entry].launch_noalloc(a, scratch, static_cast<uint32_t>(splits));
}

}  // namespace tcab
