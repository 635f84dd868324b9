// reduce_outer.cu -- reduce t[b, k, c] over the MIDDLE axis k in one pass:
// sum (fp32), max (fp32) and argmax (int32, lowest index among equal maxima).
//
// This is the class of the reference's middle-axis kernels (the reduced axis is
// parked last by `as`: testing/kernels/runtime/row_sum.tca:18-33, emitted form
// internal/cg/cxx/testdata/bracket_amort.cu:7-78 with per-thread Frag
// accumulators). There, one thread walks the reduced axis of one output with
// scalar loads; here a warp reads 512 contiguous bytes of one k-row per load
// instruction and the k axis is split over the warps of the CTA.
//
// Layout: a CTA owns (one b, a tile of 32*V*CV columns). Lane l owns CV vectors
// of V columns; warp w owns k = w, w+KW, w+2*KW, ... The per-thread state is
// (sum, best, best_index) per owned column. Each thread issues UNROLL
// independent 16-byte loads before folding them, so a CTA keeps
// 32*KW*UNROLL*CV*16 bytes in flight. The KW partial states per column are then
// combined through shared memory in ascending warp order with the tie rule
// "greater value, or equal value and lower index", which makes max and argmax
// bit-exact against a sequential ascending fold with a strict `>` update.
// Algorithmic bytes: 4 per input element plus 12 per output column.
//
// Few columns and a long k (column statistics of a tall matrix) leave fewer tiles than SMs. The k axis
// is then also split over CTAs: each writes its partial (sum, best, best_index) per column to a scratch
// buffer and a second small kernel folds the partials in ascending split order with the same tie rule.
#include <map>
#include <mutex>
#include <utility>

#include "common.cuh"

namespace tcab {
namespace {

template <int V>
struct ColVec;
template <>
struct ColVec<4> {
  static __device__ __forceinline__ void load(const float* p, float* f) {
    const float4 q = ld_stream(reinterpret_cast<const float4*>(p));
    f[0] = q.x; f[1] = q.y; f[2] = q.z; f[3] = q.w;
  }
};
template <>
struct ColVec<1> {
  static __device__ __forceinline__ void load(const float* p, float* f) { f[0] = ld_stream(p); }
};

template <int V, int CV, int KW, int UNROLL>
__global__ void __launch_bounds__(32 * KW)
reduce_outer_kernel(const float* __restrict__ t, float* __restrict__ sum, float* __restrict__ mx,
                    int32_t* __restrict__ amax, uint32_t nb, uint32_t nk, uint32_t nc,
                    uint32_t tiles_per_b, uint32_t ksplit, uint32_t klen, float* __restrict__ part) {
  constexpr int TILE_C = 32 * V * CV;
  constexpr int NCOL = V * CV;  // columns owned by a thread
  extern __shared__ float smem[];
  float* s_sum = smem;                                   // [KW][TILE_C]
  float* s_max = smem + KW * TILE_C;                     // [KW][TILE_C]
  int32_t* s_idx = reinterpret_cast<int32_t*>(smem + 2 * KW * TILE_C);  // [KW][TILE_C]

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

  for (uint32_t work = blockIdx.x; work < nb * tiles_per_b * ksplit; work += gridDim.x) {
    const uint32_t tile = work / ksplit, ks = work % ksplit;  // ks: which range of k (one range unless split)
    const uint32_t b = tile / tiles_per_b;
    const uint32_t c0 = (tile % tiles_per_b) * TILE_C;
    const float* base = t + static_cast<size_t>(b) * nk * nc;
    const uint32_t kbeg = ks * klen, kend = min(nk, kbeg + klen);

    float acc[NCOL], best[NCOL];
    int32_t bidx[NCOL];
#pragma unroll
    for (int j = 0; j < NCOL; ++j) {
      acc[j] = 0.0f;
      best[j] = -INFINITY;
      bidx[j] = 0;
    }
    // Column of vector i of this lane: c0 + (i*32 + lane)*V
    bool colok[CV];
#pragma unroll
    for (int i = 0; i < CV; ++i) colok[i] = c0 + (i * 32 + lane) * V < nc;  // nc % V == 0 when V == 4

    for (uint32_t k0 = kbeg + warp; k0 < kend; k0 += KW * UNROLL) {
      float f[UNROLL][NCOL];
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const uint32_t k = k0 + u * KW;
#pragma unroll
        for (int i = 0; i < CV; ++i) {
          if (k < kend && colok[i]) {
            ColVec<V>::load(base + static_cast<size_t>(k) * nc + c0 + (i * 32 + lane) * V, &f[u][i * V]);
          } else {
#pragma unroll
            for (int j = 0; j < V; ++j) f[u][i * V + j] = 0.0f;
          }
        }
      }
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const uint32_t k = k0 + u * KW;
        if (k < kend) {
#pragma unroll
          for (int j = 0; j < NCOL; ++j) {
            const float v = f[u][j];
            acc[j] += v;
            if (v > best[j]) {  // strict: the lowest index among equals survives
              best[j] = v;
              bidx[j] = static_cast<int32_t>(k);
            }
          }
        }
      }
    }

#pragma unroll
    for (int i = 0; i < CV; ++i)
#pragma unroll
      for (int j = 0; j < V; ++j) {
        const int col = (i * 32 + lane) * V + j;
        s_sum[warp * TILE_C + col] = acc[i * V + j];
        s_max[warp * TILE_C + col] = best[i * V + j];
        s_idx[warp * TILE_C + col] = bidx[i * V + j];
      }
    __syncthreads();
    for (int col = threadIdx.x; col < TILE_C; col += 32 * KW) {
      if (c0 + col < nc) {
        float a = 0.0f, bv = -INFINITY;
        int32_t bi = 0;
#pragma unroll
        for (int w = 0; w < KW; ++w) {
          a += s_sum[w * TILE_C + col];
          const float v = s_max[w * TILE_C + col];
          const int32_t vi = s_idx[w * TILE_C + col];
          // a warp that saw no k (nk < KW) still holds (-inf, 0): never preferred over a real entry,
          // and equal to the initial state otherwise
          if (v > bv || (v == bv && vi < bi)) {
            bv = v;
            bi = vi;
          }
        }
        const size_t o = static_cast<size_t>(b) * nc + c0 + col;
        if (ksplit > 1) {  // partial state of this k range: [3][ksplit][nb * nc]
          const size_t plane = static_cast<size_t>(ksplit) * nb * nc, po = static_cast<size_t>(ks) * nb * nc + o;
          part[po] = a;
          part[plane + po] = bv;
          part[2 * plane + po] = __int_as_float(bi);
        } else {
          if (sum) sum[o] = a;
          if (mx) mx[o] = bv;
          if (amax) amax[o] = bi;
        }
      }
    }
    __syncthreads();  // shared memory is rewritten by the next tile
  }
}

// The same reduction with a WARP per (b, column tile), for narrow rows (most lanes of a CTA's column tile would own
// no column) and short reduced axes (a CTA per tile would do a few hundred bytes of work between two barriers). A
// lane loads V columns at once (4: 16-byte vectors; 1: any nc and alignment). The lanes cover g column groups of V
// and 32 / g consecutive k rows per step (contiguous in memory when the tile is the whole row; lanes beyond
// g * (32 / g) idle); a lane folds the rows it sees in ascending order, lanes with the same column group then meet
// by shuffles under the same rule -- greater value, or equal value and lower index -- and lanes 0..g-1 store. No
// shared memory, no barrier.
template <int UNROLL, int V>
__global__ void __launch_bounds__(256)
reduce_outer_flat(const float* __restrict__ t, float* __restrict__ sum, float* __restrict__ mx, int32_t* __restrict__ amax,
                  uint32_t nb, uint32_t nk, uint32_t nc, uint32_t tiles_per_b, uint32_t g, uint32_t ksplit, uint32_t klen,
                  float* __restrict__ part) {
  // ksplit > 1 (few tiles, a long reduced axis): a CTA takes range blockIdx % ksplit of klen rows of ONE (b, column
  // tile); its eight warps interleave step by step, so that the CTA streams one contiguous piece of memory, meet in
  // shared memory, and the CTA writes its state to part[3][ksplit][nb * nc] for reduce_outer_finish.
  const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint64_t work;
  uint32_t kbeg = 0, kend = nk, kstep = (32 / g) * UNROLL, ks = 0;
  if (ksplit > 1) {
    work = blockIdx.x / ksplit;
    ks = blockIdx.x % ksplit;
    const uint32_t first = ks * klen < nk ? ks * klen : nk;  // a range that would start past the end is empty
    kend = nk - first < klen ? nk : first + klen;
    kbeg = first + warp * kstep;
    if (kbeg > kend) kbeg = kend;
    kstep *= 8;
  } else {
    work = static_cast<uint64_t>(blockIdx.x) * 8 + warp;
    if (work >= static_cast<uint64_t>(nb) * tiles_per_b) return;  // the whole warp leaves
  }
  const uint32_t b = static_cast<uint32_t>(work / tiles_per_b), tile = static_cast<uint32_t>(work % tiles_per_b);
  const uint32_t rows_per_step = 32 / g;
  const uint32_t cg = lane % g, kr = lane / g;
  const uint32_t col = tile * (32 * V) + cg * V;  // g < 32 only when one tile is the whole row
  const bool colok = col < nc && kr < rows_per_step;
  const float* base = t + static_cast<size_t>(b) * nk * nc + col;

  float acc[V], best[V];
  int32_t bidx[V];
#pragma unroll
  for (int j = 0; j < V; ++j) {
    acc[j] = 0.0f;
    best[j] = -INFINITY;
    bidx[j] = 0;
  }
  if (colok) {
    uint32_t k0 = kbeg + kr;
    const size_t ustride = static_cast<size_t>(rows_per_step) * nc;
    // Iterations whose UNROLL rows all exist: no predicates. With 4-byte loads the running maximum meets the maximum
    // of the iteration's rows instead of every row -- a new maximum is rare after the first few rows, and only then is
    // the row looked up (the first one that holds it, so the lowest index among equals survives as below).
    for (; kend > (UNROLL - 1) * rows_per_step && k0 < kend - (UNROLL - 1) * rows_per_step; k0 += kstep) {
      float f[UNROLL][V];
      const float* at = base + static_cast<size_t>(k0) * nc;
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) ColVec<V>::load(at + u * ustride, f[u]);
      if constexpr (V == 1) {  // 16 rows of one column per iteration
        float m = f[0][0];
        acc[0] += f[0][0];
#pragma unroll
        for (int u = 1; u < UNROLL; ++u) {
          acc[0] += f[u][0];
          m = fmaxf(m, f[u][0]);  // ignores NaN, as a comparison does
        }
        if (m > best[0]) {
          int first = UNROLL - 1;
#pragma unroll
          for (int u = UNROLL - 2; u >= 0; --u) first = f[u][0] == m ? u : first;
#pragma unroll
          for (int u = 0; u < UNROLL; ++u)
            if (u == first) best[0] = f[u][0];  // the element itself: -0.0 and 0.0 compare equal
          bidx[0] = static_cast<int32_t>(k0 + first * rows_per_step);
        }
      } else {  // four rows of four columns: comparing every element is cheaper than the detour (measured)
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
#pragma unroll
          for (int j = 0; j < V; ++j) {
            const float v = f[u][j];
            acc[j] += v;
            if (v > best[j]) {  // strict: the lowest index among equals survives
              best[j] = v;
              bidx[j] = static_cast<int32_t>(k0 + u * rows_per_step);
            }
          }
        }
      }
    }
    for (; k0 < kend; k0 += kstep) {  // the ragged end of this lane's rows
      float f[UNROLL][V];
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const uint32_t k = k0 + u * rows_per_step;
        if (k < kend) ColVec<V>::load(base + static_cast<size_t>(k) * nc, f[u]);
      }
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const uint32_t k = k0 + u * rows_per_step;
        if (k < kend) {
#pragma unroll
          for (int j = 0; j < V; ++j) {
            const float v = f[u][j];
            acc[j] += v;
            if (v > best[j]) {  // strict: the lowest index among equals survives
              best[j] = v;
              bidx[j] = static_cast<int32_t>(k);
            }
          }
        }
      }
    }
  }
  if ((g & (g - 1)) == 0) {
    for (uint32_t off = 16; off >= g; off >>= 1) {
#pragma unroll
      for (int j = 0; j < V; ++j) {
        acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], off);
        const float v = __shfl_xor_sync(0xffffffffu, best[j], off);
        const int32_t vi = __shfl_xor_sync(0xffffffffu, bidx[j], off);
        if (v > best[j] || (v == best[j] && vi < bidx[j])) {  // a lane that saw no row holds (-inf, 0): the initial state
          best[j] = v;
          bidx[j] = vi;
        }
      }
    }
  } else {  // lanes cg, cg + g, cg + 2 g, ... hold column group cg: lanes 0..g-1 collect them
    for (uint32_t r = 1; r < rows_per_step; ++r) {
      const uint32_t src = (lane + r * g) & 31;
#pragma unroll
      for (int j = 0; j < V; ++j) {
        const float a = __shfl_sync(0xffffffffu, acc[j], src);
        const float v = __shfl_sync(0xffffffffu, best[j], src);
        const int32_t vi = __shfl_sync(0xffffffffu, bidx[j], src);
        if (lane < g) {
          acc[j] += a;
          if (v > best[j] || (v == best[j] && vi < bidx[j])) {
            best[j] = v;
            bidx[j] = vi;
          }
        }
      }
    }
  }
  if (ksplit > 1) {
    __shared__ float s_sum[8][128], s_max[8][128];
    __shared__ int32_t s_idx[8][128];
    if (lane < g) {
#pragma unroll
      for (int j = 0; j < V; ++j) {
        s_sum[warp][cg * V + j] = acc[j];
        s_max[warp][cg * V + j] = best[j];
        s_idx[warp][cg * V + j] = bidx[j];
      }
    }
    __syncthreads();
    const uint32_t c = threadIdx.x, tile_col = tile * (32 * V) + c;
    if (c < V * g && tile_col < nc) {
      float a = 0.0f, bv = -INFINITY;
      int32_t bi = 0x7fffffff;
#pragma unroll
      for (int w = 0; w < 8; ++w) {
        a += s_sum[w][c];
        const float v = s_max[w][c];
        const int32_t vi = s_idx[w][c];
        if (v > bv || (v == bv && vi < bi)) {
          bv = v;
          bi = vi;
        }
      }
      const size_t cells = static_cast<size_t>(nb) * nc, plane = ksplit * cells;
      const size_t po = ks * cells + static_cast<size_t>(b) * nc + tile_col;
      part[po] = a;
      part[plane + po] = bv;
      part[2 * plane + po] = __int_as_float(bi);
    }
    return;
  }
  if (lane < g && colok) {
    const size_t o = static_cast<size_t>(b) * nc + col;
#pragma unroll
    for (int j = 0; j < V; ++j) {
      if (sum) sum[o + j] = acc[j];
      if (mx) mx[o + j] = best[j];
      if (amax) amax[o + j] = bidx[j];
    }
  }
}

// Folds the partial states of the k ranges under the rule of the cross-warp combine above -- greater value, or equal
// value and lower index -- so the lowest index among equal maxima survives whichever range it came from. `lanes` (a
// power of two up to 32) threads share a cell: each folds every lanes-th state in ascending order, then they meet by
// shuffles.
__global__ void __launch_bounds__(256)
reduce_outer_finish(const float* __restrict__ part, float* __restrict__ sum, float* __restrict__ mx,
                    int32_t* __restrict__ amax, uint32_t cells, uint32_t ksplit, uint32_t lanes) {
  const uint32_t t = blockIdx.x * 256 + threadIdx.x;
  const uint32_t o = t / lanes, l = t % lanes;
  const size_t plane = static_cast<size_t>(ksplit) * cells;
  float a = 0.0f, bv = -INFINITY;
  int32_t bi = 0x7fffffff;  // no state seen yet: any real index is lower
  if (o < cells) {
#pragma unroll 4
    for (uint32_t ks = l; ks < ksplit; ks += lanes) {
      const size_t po = static_cast<size_t>(ks) * cells + o;
      a += part[po];
      const float v = part[plane + po];
      const int32_t vi = __float_as_int(part[2 * plane + po]);
      if (v > bv || (v == bv && vi < bi)) {
        bv = v;
        bi = vi;
      }
    }
  }
  for (uint32_t off = lanes >> 1; off > 0; off >>= 1) {
    a += __shfl_xor_sync(0xffffffffu, a, off);
    const float v = __shfl_xor_sync(0xffffffffu, bv, off);
    const int32_t vi = __shfl_xor_sync(0xffffffffu, bi, off);
    if (v > bv || (v == bv && vi < bi)) {
      bv = v;
      bi = vi;
    }
  }
  if (o < cells && l == 0) {
    if (sum) sum[o] = a;
    if (mx) mx[o] = bv;
    if (amax) amax[o] = bi;
  }
}

// Scratch for the partial states: kMaxPartialCells cells x 3 values per (device, stream), allocated the
// first time a stream needs the split (stream_scratch).
constexpr uint32_t kMaxPartialCells = 262144;  // ksplit * nb * nc at most: 3 MiB
float* outer_scratch(cudaStream_t stream) {
  return static_cast<float*>(
      stream_scratch(kScratchOuter, stream, static_cast<size_t>(3) * kMaxPartialCells * sizeof(float), false));
}

// How many CTAs share the k axis of one (b, column tile): none while the tiles alone fill the GPU; otherwise as
// many as make the whole grid resident at once (`resident` = CTAs of this kernel the GPU holds: one wave, no
// tail), each with at least 256 k, within the scratch.
uint32_t choose_ksplit(uint64_t tiles, uint32_t nb, uint32_t nk, uint32_t nc, uint64_t resident, int forced) {
  const uint64_t cells = static_cast<uint64_t>(nb) * nc;
  if (cells == 0 || cells > kMaxPartialCells) return 1;
  uint64_t want;
  if (forced > 0) {
    want = static_cast<uint64_t>(forced);
  } else {
    if (tiles * 2 > resident || tiles >= 4 * static_cast<uint64_t>(sm_count())) return 1;  // as plan_outer_splits
    want = resident / tiles;
    if (want > nk / 256) want = nk / 256;
  }
  if (want > kMaxPartialCells / cells) want = kMaxPartialCells / cells;
  if (want > nk) want = nk;
  return want < 2 ? 1 : static_cast<uint32_t>(want);
}

int launch_finish(const float* part, float* sum, float* mx, int32_t* amax, uint32_t cells, uint32_t states, cudaStream_t s) {
  const uint32_t lanes = finish_lanes(states);
  const uint64_t threads = static_cast<uint64_t>(cells) * lanes;
  reduce_outer_finish<<<static_cast<unsigned>((threads + 255) / 256), 256, 0, s>>>(part, sum, mx, amax, cells, states, lanes);
  count_launch();
  return check_launch("reduce_outer_finish");
}

template <int V, int CV, int KW, int UNROLL>
int launch(const float* t, float* sum, float* mx, int32_t* amax, uint32_t nb, uint32_t nk, uint32_t nc,
           int ctas_per_sm, int forced_ksplit, cudaStream_t s) {
  constexpr int TILE_C = 32 * V * CV;
  constexpr int THREADS = 32 * KW;
  const size_t smem = static_cast<size_t>(3) * KW * TILE_C * sizeof(float);
  auto* fn = reduce_outer_kernel<V, CV, KW, UNROLL>;
  if (smem > 48 * 1024) {
    if (cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess)
      return fail(TCAB_ERR_CUDA, "reduce_outer: cannot reserve %zu bytes of shared memory", smem);
  }
  const uint32_t tiles_per_b = (nc + TILE_C - 1) / TILE_C;
  const uint64_t tiles = static_cast<uint64_t>(nb) * tiles_per_b;
  const int occ = occupancy(reinterpret_cast<const void*>(fn), THREADS, smem);
  uint32_t ksplit = choose_ksplit(tiles, nb, nk, nc, static_cast<uint64_t>(occ > 0 ? occ : 1) * sm_count(), forced_ksplit);
  float* part = ksplit > 1 ? outer_scratch(s) : nullptr;
  if (part == nullptr) ksplit = 1;
  const uint32_t klen = ksplit > 1 ? (nk + ksplit - 1) / ksplit : nk;
  const uint64_t work = tiles * ksplit;
  // one CTA per unit of work unless the tuning hook caps the grid (the loop in the kernel then takes over)
  uint64_t grid = ctas_per_sm > 0 ? static_cast<uint64_t>(sm_count()) * ctas_per_sm : work;
  if (grid > work) grid = work;
  if (grid > 0x7fffffffull) grid = 0x7fffffffull;
  fn<<<static_cast<unsigned>(grid), THREADS, smem, s>>>(t, sum, mx, amax, nb, nk, nc, tiles_per_b, ksplit, klen, part);
  count_launch();
  int rc = check_launch("reduce_outer_kernel");
  if (rc != TCAB_OK || ksplit == 1) return rc;
  return launch_finish(part, sum, mx, amax, nb * nc, ksplit, s);
}

}  // namespace

int launch_reduce_outer(const float* t, float* sum, float* mx, int32_t* amax, uint32_t nb, uint32_t nk,
                        uint32_t nc, cudaStream_t s) {
  if (nb == 0 || nc == 0) return TCAB_OK;
  if (static_cast<uint64_t>(nb) * ((nc + 31) / 32) > 0xffffffffull)
    return fail(TCAB_ERR_TOO_LARGE, "reduce_outer: too many column tiles");
  const bool vec = (nc % 4 == 0) && aligned16(t);
  const Tune& tn = tune(kReduceOuter);
  // p0: vectors per lane (1|2), p1: warps splitting k (4|8|16), p2: CTAs per SM, p3: CTAs splitting k (forced).
  const int cv = tn.p0 > 0 ? tn.p0 : 1;
  const int kw = tn.p1 > 0 ? tn.p1 : 8;
  // narrow rows, short reduced axes: a warp per (b, column tile); p1 == 1 takes the warps whatever the shape
  if (tn.p0 <= 0 && (tn.p1 <= 0 || tn.p1 == 1) && tn.p3 <= 0) {
    const uint32_t g = tn.p1 == 1 ? outer_flat_width(nc, vec) : outer_flat_groups(nb, nk, nc, sm_count(), vec);
    if (g != 0) {
      const uint32_t tile = vec ? 128 : 32;
      const uint32_t tiles_per_b = (nc + tile - 1) / tile;
      const uint64_t work = static_cast<uint64_t>(nb) * tiles_per_b;
      uint32_t klen = nk;
      uint32_t ksplit = outer_flat_ranges(nb, nk, nc, g, vec, sm_count(), kMaxPartialCells, &klen);
      float* part = ksplit > 1 ? outer_scratch(s) : nullptr;
      if (part == nullptr) {
        ksplit = 1;
        klen = nk;
      }
      const uint64_t grid = ksplit > 1 ? work * ksplit : (work + 7) / 8;  // a CTA per range, or eight tiles per CTA
      if (vec) {
        reduce_outer_flat<4, 4><<<static_cast<unsigned>(grid), 256, 0, s>>>(t, sum, mx, amax, nb, nk, nc, tiles_per_b, g,
                                                                            ksplit, klen, part);
      } else {  // 4-byte loads need more of them in flight for the same bytes
        reduce_outer_flat<16, 1><<<static_cast<unsigned>(grid), 256, 0, s>>>(t, sum, mx, amax, nb, nk, nc, tiles_per_b, g,
                                                                             ksplit, klen, part);
      }
      count_launch();
      int rc = check_launch("reduce_outer_flat");
      if (rc != TCAB_OK || ksplit == 1) return rc;
      return launch_finish(part, sum, mx, amax, nb * nc, ksplit, s);
    }
  }
  if (vec) {
    if (cv == 1 && kw == 8) return launch<4, 1, 8, 4>(t, sum, mx, amax, nb, nk, nc, tn.p2, tn.p3, s);
    if (cv == 2 && kw == 8) return launch<4, 2, 8, 4>(t, sum, mx, amax, nb, nk, nc, tn.p2, tn.p3, s);
    if (cv == 1 && kw == 16) return launch<4, 1, 16, 4>(t, sum, mx, amax, nb, nk, nc, tn.p2, tn.p3, s);
    if (cv == 2 && kw == 16) return launch<4, 2, 16, 2>(t, sum, mx, amax, nb, nk, nc, tn.p2, tn.p3, s);
    if (cv == 1 && kw == 4) return launch<4, 1, 4, 8>(t, sum, mx, amax, nb, nk, nc, tn.p2, tn.p3, s);
    if (cv == 2 && kw == 4) return launch<4, 2, 4, 4>(t, sum, mx, amax, nb, nk, nc, tn.p2, tn.p3, s);
    return fail(TCAB_ERR_UNSUPPORTED, "reduce_outer: no kernel for tuned shape %d x %d", cv, kw);
  }
  return launch<1, 1, 8, 4>(t, sum, mx, amax, nb, nk, nc, tn.p2, tn.p3, s);
}

}  // namespace tcab
