// chain_kernels.cuh -- map | reduce | map chains over one axis, generic in the lambdas.
//
// Self-contained device code (no includes): the same text is compiled ahead of
// time with the precompiled lambdas (chain_reduce.cu) and at run time with a
// lambda printed from the caller's expression (the run-time compiler prepends
// nothing but the two functor structs).
//
// The kernels replace the reference's emitted reduce kernels
// (internal/cg/cxx/testdata/reduce_warp.cu:12-62, reduce_splitk.cu:13-80,
// bracket_amort.cu:7-78) and its reducer brackets (runtime/tca/reducer.h:36-181):
// every thread folds its share of the reduced axis in registers and the partials
// meet in ONE tree per output, instead of one shuffle tree and two barriers per
// reduced ELEMENT. Padded points never reach the map lambda (design/tca.md:297-299);
// an empty reduction returns init (design/tca.md:299).
//
// Functor contract:
//   struct Map  { static __device__ float apply(const float* p, const float* c); }  p[i] = operand i
//   struct Post { static __device__ float apply(const float* p, const float* c); }  p[0] = reduced value
// COMBINE: 0 = p0 + p1, 1 = fmaxf(p0, p1), 2 = fminf(p0, p1).
// Operands travel to the functor as 32-bit registers: an f32 operand as its value, an i32 / u32 operand as
// its bit pattern, a bf16 operand widened to f32 at the load (exact). The functor's prologue gives each p#
// its declared type back (the run-time compiler prints that prologue from the operands' element types), and
// a map-only functor returns its result the same way. BF is the bit mask of the operands that are bf16 in
// memory: those are read with 8-byte (four elements) or 2-byte loads.
#pragma once

namespace tcabk {

typedef unsigned int u32;
typedef unsigned long long u64;

constexpr int kMaxCaptures = 16;  // user captures plus lifted literals

template <int NIN>
struct Ptrs {
  const float* p[NIN];
};
struct Caps {
  float c[kMaxCaptures];
};

template <int COMBINE>
struct Comb;
template <>
struct Comb<0> {
  static __device__ __forceinline__ float identity() { return 0.0f; }
  static __device__ __forceinline__ float apply(float a, float b) { return a + b; }
};
template <>
struct Comb<1> {
  static __device__ __forceinline__ float identity() { return -__int_as_float(0x7f800000); }
  static __device__ __forceinline__ float apply(float a, float b) { return fmaxf(a, b); }
};
template <>
struct Comb<2> {
  static __device__ __forceinline__ float identity() { return __int_as_float(0x7f800000); }
  static __device__ __forceinline__ float apply(float a, float b) { return fminf(a, b); }
};

struct PostNone {
  static __device__ __forceinline__ float apply(const float* p, const float*) { return p[0]; }
};

template <int V>
struct Ld;
template <>
struct Ld<4> {
  static __device__ __forceinline__ void load(const float* base, u64 vec_index, float* f) {
    const float4 q = __ldcs(reinterpret_cast<const float4*>(base) + vec_index);
    f[0] = q.x; f[1] = q.y; f[2] = q.z; f[3] = q.w;
  }
};
template <>
struct Ld<1> {
  static __device__ __forceinline__ void load(const float* base, u64 vec_index, float* f) {
    f[0] = __ldcs(base + vec_index);
  }
};

// bf16 in memory: the top half of an f32 (widening is exact). Kept free of cuda_bf16.h so that this text also
// compiles at run time without any include path.
__device__ __forceinline__ float bf16_bits_to_float(unsigned int h) { return __uint_as_float(h << 16); }
__device__ __forceinline__ unsigned int float_to_bf16_bits(float f) {  // round to nearest even, quiet NaN kept
  // the conversion instruction rounds to nearest even and keeps infinities; it turns every NaN into 0x7fff, so a NaN
  // is written here with its sign and payload, quieted (in integer arithmetic this function was eight instructions
  // per value, and a chain over bf16 operands was bound by them, not by memory)
  unsigned short h;
  asm("cvt.rn.bf16.f32 %0, %1;" : "=h"(h) : "f"(f));
  if (f != f) h = static_cast<unsigned short>((__float_as_uint(f) >> 16) | 0x0040u);
  return h;
}
// Two values at once with the conversion instruction (round to nearest even, as above); it turns every NaN into
// 0x7fff, so a NaN is put back as float_to_bf16_bits writes it (sign and payload kept, quieted).
__device__ __forceinline__ unsigned int pack_bf16x2(float lo, float hi) {
  unsigned int d;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
  if (lo != lo) d = (d & 0xffff0000u) | ((__float_as_uint(lo) >> 16) | 0x0040u);
  if (hi != hi) d = (d & 0x0000ffffu) | (((__float_as_uint(hi) >> 16) | 0x0040u) << 16);
  return d;
}
struct bf16 {  // the value type a bf16 operand has inside a lambda: convertible, not arithmetic
  // kept WIDENED (an f32 whose low 16 bits are zero): operands arrive that way from the kernels' loads and leave
  // that way for their stores, so converting to and from f32 inside a lambda costs nothing; only bf16(f32) rounds
  float w;
  __device__ __forceinline__ bf16() : w(0.0f) {}
  __device__ __forceinline__ explicit bf16(float f) : w(bf16_bits_to_float(float_to_bf16_bits(f))) {}
  // from the f32 register a kernel widened a bf16 operand into: nothing to round
  static __device__ __forceinline__ bf16 widened(float f) {
    bf16 r;
    r.w = f;
    return r;
  }
  __device__ __forceinline__ explicit operator float() const { return w; }
  __device__ __forceinline__ explicit operator int() const { return static_cast<int>(w); }
  __device__ __forceinline__ explicit operator unsigned int() const { return static_cast<unsigned int>(w); }
};

// Operand `a` of a kernel: element size by the BF mask. `index` counts vectors of V elements.
template <int V, bool IS_BF16>
struct LdT;
template <>
struct LdT<4, false> {
  static __device__ __forceinline__ void load(const float* base, u64 index, float* f) { Ld<4>::load(base, index, f); }
};
template <>
struct LdT<1, false> {
  static __device__ __forceinline__ void load(const float* base, u64 index, float* f) { Ld<1>::load(base, index, f); }
};
template <>
struct LdT<4, true> {
  static __device__ __forceinline__ void load(const float* base, u64 index, float* f) {
    const uint2 q = __ldcs(reinterpret_cast<const uint2*>(base) + index);
    f[0] = bf16_bits_to_float(q.x & 0xffffu); f[1] = bf16_bits_to_float(q.x >> 16);
    f[2] = bf16_bits_to_float(q.y & 0xffffu); f[3] = bf16_bits_to_float(q.y >> 16);
  }
};
template <>
struct LdT<1, true> {
  static __device__ __forceinline__ void load(const float* base, u64 index, float* f) {
    f[0] = bf16_bits_to_float(__ldcs(reinterpret_cast<const unsigned short*>(base) + index));
  }
};
// Vectors of eight: one 16-byte load of a bf16 operand (chains whose operands are all bf16 would otherwise move 8 bytes
// per load and reach their thresholds, which count vectors, at half the bytes), two of an f32 operand.
template <>
struct LdT<8, true> {
  static __device__ __forceinline__ void load(const float* base, u64 index, float* f) {
    const uint4 q = __ldcs(reinterpret_cast<const uint4*>(base) + index);
    const unsigned int w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      f[2 * i] = __uint_as_float(w[i] << 16);
      f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
};
template <>
struct LdT<8, false> {
  static __device__ __forceinline__ void load(const float* base, u64 index, float* f) {
    Ld<4>::load(base, 2 * index, f);
    Ld<4>::load(base, 2 * index + 1, f + 4);
  }
};
template <int V, int BF, int A>
__device__ __forceinline__ void load_operand(const float* base, u64 index, float* f) {
  LdT<V, ((BF >> A) & 1) != 0>::load(base, index, f);
}
// The NIN operands at one vector index (compile-time operand numbers select the element size).
template <int V, int BF, int NIN, int A = 0>
struct LoadAll {
  static __device__ __forceinline__ void at(const float* const* p, u64 index, float (*f)[V]) {
    load_operand<V, BF, A>(p[A], index, f[A]);
    LoadAll<V, BF, NIN, A + 1>::at(p, index, f);
  }
};
template <int V, int BF, int NIN>
struct LoadAll<V, BF, NIN, NIN> {
  static __device__ __forceinline__ void at(const float* const*, u64, float (*)[V]) {}
};

// Middle-axis reductions: operands at vector index `index` of the [nb, nk, nc] tensors, except those of the
// mask CELL, which have ONE value per output cell (shape [nb, 1, nc]: they lack the reduced axis) and were
// loaded once, before the k loop, into cellval.
template <int V, int BF, int CELL, int NIN, int A = 0>
struct LoadOuterAll {
  static __device__ __forceinline__ void at(const float* const* p, u64 index, const float (*cellval)[V], float (*f)[V]) {
    if constexpr (((CELL >> A) & 1) != 0) {
#pragma unroll
      for (int j = 0; j < V; ++j) f[A][j] = cellval[A][j];
    } else {
      load_operand<V, BF, A>(p[A], index, f[A]);
    }
    LoadOuterAll<V, BF, CELL, NIN, A + 1>::at(p, index, cellval, f);
  }
  static __device__ __forceinline__ void cells(const float* const* p, u64 cell_index, float (*cellval)[V]) {
    if constexpr (((CELL >> A) & 1) != 0) load_operand<V, BF, A>(p[A], cell_index, cellval[A]);
    LoadOuterAll<V, BF, CELL, NIN, A + 1>::cells(p, cell_index, cellval);
  }
};
template <int V, int BF, int CELL, int NIN>
struct LoadOuterAll<V, BF, CELL, NIN, NIN> {
  static __device__ __forceinline__ void at(const float* const*, u64, const float (*)[V], float (*)[V]) {}
  static __device__ __forceinline__ void cells(const float* const*, u64, float (*)[V]) {}
};

template <class C, int WIDTH>
__device__ __forceinline__ float lanes_allreduce(float v) {
#pragma unroll
  for (int off = WIDTH / 2; off > 0; off >>= 1) v = C::apply(v, __shfl_xor_sync(0xffffffffu, v, off));
  return v;
}

__host__ __device__ constexpr int inner_cta_threads(int tpr) { return tpr > 128 ? tpr : 128; }

// Operands that are not indexed by every iteration axis (the reference's structural indexing lets an operand
// bind a subset of the live axes, pkg/chain.go checkOperand: x[i] inside an (i, j) iteration): RB is the bit
// mask of operands with ONE value per row (shape [rows, 1]: a max or a sum from an earlier statement), CB of
// operands with one row shared by all rows (shape [1, cols]: a bias, gamma, beta). A row value is loaded
// once per row and thread, a shared row with the same vector index in every row (it stays in L1 / L2).
template <int V, int BF, int RB, int CB, int NIN, int A = 0>
struct LoadRowAll {
  static __device__ __forceinline__ void at(const float* const* p, u64 row, u32 nvec, u32 idx, const float* rowval,
                                            float (*f)[V]) {
    if constexpr (((RB >> A) & 1) != 0) {
#pragma unroll
      for (int j = 0; j < V; ++j) f[A][j] = rowval[A];
    } else if constexpr (((CB >> A) & 1) != 0) {
      load_operand<V, BF, A>(p[A], idx, f[A]);
    } else {
      load_operand<V, BF, A>(p[A], row * nvec + idx, f[A]);
    }
    LoadRowAll<V, BF, RB, CB, NIN, A + 1>::at(p, row, nvec, idx, rowval, f);
  }
  static __device__ __forceinline__ void row_values(const float* const* p, u64 row, float* rowval) {
    if constexpr (((RB >> A) & 1) != 0) LdT<1, ((BF >> A) & 1) != 0>::load(p[A], row, &rowval[A]);
    LoadRowAll<V, BF, RB, CB, NIN, A + 1>::row_values(p, row, rowval);
  }
};
template <int V, int BF, int RB, int CB, int NIN>
struct LoadRowAll<V, BF, RB, CB, NIN, NIN> {
  static __device__ __forceinline__ void at(const float* const*, u64, u32, u32, const float*, float (*)[V]) {}
  static __device__ __forceinline__ void row_values(const float* const*, u64, float*) {}
};

// One thread's share of a row: vectors t, t + TPR, ... of the row's nvec vectors.
template <class Map, class C, int NIN, int TPR, int V, int BF, int RB = 0, int CB = 0>
__device__ __forceinline__ float fold_row_share(const float* const* p, u64 row, u32 nvec, int t, const float* caps) {
  float acc = C::identity();
  float rowval[NIN];
  LoadRowAll<V, BF, RB, CB, NIN>::row_values(p, row, rowval);
#pragma unroll(V == 1 ? 16 : 8)
  for (u32 idx = t; idx < nvec; idx += TPR) {
    float f[NIN][V];
    LoadRowAll<V, BF, RB, CB, NIN>::at(p, row, nvec, idx, rowval, f);
#pragma unroll
    for (int j = 0; j < V; ++j) {
      float v[NIN];
#pragma unroll
      for (int a = 0; a < NIN; ++a) v[a] = f[a][j];
      acc = C::apply(acc, Map::apply(v, caps));
    }
  }
  return acc;
}

// The same for rows that are not whole 16-byte vectors although the operands are aligned (nk % 4 != 0): a row then
// starts 0 ... 3 elements before a vector boundary. The thread takes the row's whole vectors as above; the up to six
// elements before the first and after the last of them go to threads 0, 1, ... one each (two with four threads),
// loaded before the vector loop so that their latency overlaps with it. TPR >= 4.
template <class Map, class C, int NIN, int TPR, int BF>
__device__ __forceinline__ float fold_row_share_ragged(const float* const* p, u64 row, u32 nk, int t, const float* caps) {
  constexpr int EDGES = TPR >= 6 ? 1 : 2;  // edge elements a thread may get
  const u64 e0 = row * nk;
  u32 head = (4u - static_cast<u32>(e0 & 3u)) & 3u;
  if (head > nk) head = nk;
  const u64 v0 = (e0 + head) >> 2;
  const u32 nfull = (nk - head) >> 2, tail = nk - head - 4 * nfull;
  float edge[EDGES][NIN][1];
#pragma unroll
  for (int q = 0; q < EDGES; ++q) {
    const u32 e = t + q * TPR;
    if (e < head + tail) LoadAll<1, BF, NIN>::at(p, e < head ? e0 + e : e0 + 4 * nfull + e, edge[q]);  // tail: e0 + head + 4 nfull + (e - head)
  }
  float acc = C::identity();
#pragma unroll 8
  for (u32 idx = t; idx < nfull; idx += TPR) {
    float f[NIN][4];
    LoadAll<4, BF, NIN>::at(p, v0 + idx, f);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float v[NIN];
#pragma unroll
      for (int a = 0; a < NIN; ++a) v[a] = f[a][j];
      acc = C::apply(acc, Map::apply(v, caps));
    }
  }
#pragma unroll
  for (int q = 0; q < EDGES; ++q) {
    if (t + q * TPR < head + tail) {
      float v[NIN];
#pragma unroll
      for (int a = 0; a < NIN; ++a) v[a] = edge[q][a][0];
      acc = C::apply(acc, Map::apply(v, caps));
    }
  }
  return acc;
}

// The partials of the TPR threads of a row group meet: every thread returns the row's fold. `slots` is
// 2 x 32 floats of shared memory, alternated by `iter` so that a slot is rewritten only after everyone read it.
template <class C, int TPR>
__device__ __forceinline__ float fold_row_group(float acc, float (*slots)[32], u32 iter) {
  if constexpr (TPR > 1 && TPR <= 32) {
    acc = lanes_allreduce<C, TPR>(acc);
  } else if constexpr (TPR > 32) {
    constexpr int NW = TPR / 32;
    float* sl = slots[iter & 1];
    acc = lanes_allreduce<C, 32>(acc);
    if ((threadIdx.x & 31) == 0) sl[threadIdx.x >> 5] = acc;
    __syncthreads();
    acc = lanes_allreduce<C, NW>(sl[threadIdx.x & (NW - 1)]);
  }
  return acc;
}

// Reduce over the INNERMOST axis: operands are [rows, nk]; a group of TPR
// threads folds one row. TPR == 1 is a plain sequential ascending fold per
// thread (bit-identical to the reference's SeqReducer order). THREADS is the CTA size: 128 (256 for a CTA
// per row) by default; small problems take 1024-thread CTAs, because a launch costs by the CTA (measured in a
// graph of dependent launches: an empty grid of 1024 x 128 threads 1.7 us, of 148 x 1024 threads 0.8 us).
// RAG: rows that are not whole vectors on aligned operands (V == 4, no broadcast operands): fold_row_share_ragged.
template <class Map, class Post, int COMBINE, int NIN, int TPR, int V, int BF = 0, int THREADS = inner_cta_threads(TPR),
          int RB = 0, int CB = 0, int RAG = 0>
__global__ void __launch_bounds__(THREADS)
chain_inner(Ptrs<NIN> ins, float* __restrict__ out, u64 rows, u32 nk, float init, Caps caps) {
  typedef Comb<COMBINE> C;
  constexpr int GROUPS = THREADS / TPR;
  __shared__ float slots[2][32];

  const int g = threadIdx.x / TPR;
  const int t = threadIdx.x % TPR;
  const u32 nvec = nk / V;
  u32 iter = 0;
  // Programmatic dependent launch: when the launcher allowed this grid to start before the previous
  // grid of the stream has finished, let the next grid begin its own launch now and wait here (before the
  // first global access that returns data) until the previous grid has finished. Both are no-ops for an
  // ordinary launch. While waiting, each row group asks the L2 to fetch its first row: a prefetch moves
  // lines from DRAM into the L2, the point where all SMs' writes meet, and returns nothing to the SM, so
  // it cannot observe a stale value even if the previous grid is still writing that row; it turns the
  // DRAM latency of a short kernel's first loads into overlap with the previous kernel's tail.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if constexpr (V == 4 && RAG == 0) {
    const u64 first = static_cast<u64>(blockIdx.x) * GROUPS + g;
    if (t == 0 && first < rows && nk >= 4) {
      const u32 bytes = nk * 4u < 65536u ? nk * 4u : 65536u;  // nk % 4 == 0 and 16-byte aligned rows on this path
#pragma unroll
      for (int a = 0; a < NIN; ++a)
        if (!(((BF | RB | CB) >> a) & 1))  // full f32 / i32 / u32 rows; bf16 rows (8-byte granules) are left to the loads
          asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(ins.p[a] + first * nk), "r"(bytes) : "memory");
    }
  }
  asm volatile("griddepcontrol.wait;" ::: "memory");

  for (u64 row0 = static_cast<u64>(blockIdx.x) * GROUPS; row0 < rows;
       row0 += static_cast<u64>(gridDim.x) * GROUPS, ++iter) {
    const u64 row = row0 + g;
    const bool live = row < rows;
    float acc = C::identity();
    if constexpr (RAG != 0) {
      if (live) acc = fold_row_share_ragged<Map, C, NIN, TPR, BF>(ins.p, row, nk, t, caps.c);
    } else {
      if (live) acc = fold_row_share<Map, C, NIN, TPR, V, BF, RB, CB>(ins.p, row, nvec, t, caps.c);  // nk % V == 0
    }
    acc = fold_row_group<C, TPR>(acc, slots, iter);
    if (live && t == 0) {
      float r[1] = {C::apply(init, acc)};
      out[row] = Post::apply(r, caps.c + 8);
    }
  }
}

// Reduce over the INNERMOST axis of SHORT rows (at most 128 vectors of four): g = 1, 2, 4 ... 32 lanes per row
// (the power of two that covers the row), one 16-byte vector per lane, 32 / g rows per warp and step, UNROLL steps
// in flight. The lanes of a warp read consecutive vectors of consecutive rows, a lane folds the four values of its
// vector, the g lanes of a row meet by xor shuffles, and the first lane of a row stores. chain_inner gives a whole
// row to one thread (up to 16 vectors: every load instruction of a warp touches 32 different rows) or to four, or
// a warp to a row of 17 ... 32 vectors and lets the CTA end after four rows; both cost more than the bytes.
template <class Map, class Post, int COMBINE, int NIN, int UNROLL, int BF = 0, int VPL = 1>
__global__ void __launch_bounds__(256)
chain_inner_flat(Ptrs<NIN> ins, float* __restrict__ out, u64 rows, u32 nvec, u32 g, float init, Caps caps) {
  // VPL > 1: rows of up to 32 * VPL vectors, a warp per row (g == 32), VPL vectors per lane
  typedef Comb<COMBINE> C;
  const u32 lane = threadIdx.x & 31;
  const u32 rows_per_step = 32 / g;
  const u32 i = lane % g, r = lane / g;  // this lane's vector inside its row, and its row inside a step
  const u64 warp_id = static_cast<u64>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  const u64 row0 = warp_id * (rows_per_step * UNROLL) + r;
  if (warp_id * (rows_per_step * UNROLL) >= rows) return;  // the whole warp leaves

  float f[UNROLL][VPL][NIN][4];
#pragma unroll
  for (int u = 0; u < UNROLL; ++u) {
    const u64 row = row0 + static_cast<u64>(u) * rows_per_step;
#pragma unroll
    for (int v = 0; v < VPL; ++v)
      if (row < rows && i + v * 32 < nvec) LoadAll<4, BF, NIN>::at(ins.p, row * nvec + i + v * 32, f[u][v]);
  }
#pragma unroll
  for (int u = 0; u < UNROLL; ++u) {
    const u64 row = row0 + static_cast<u64>(u) * rows_per_step;
    float acc = C::identity();
#pragma unroll
    for (int v = 0; v < VPL; ++v) {
      if (row < rows && i + v * 32 < nvec) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float p[NIN];
#pragma unroll
          for (int a = 0; a < NIN; ++a) p[a] = f[u][v][a][j];
          acc = C::apply(acc, Map::apply(p, caps.c));
        }
      }
    }
    for (u32 off = g >> 1; off > 0; off >>= 1) acc = C::apply(acc, __shfl_xor_sync(0xffffffffu, acc, off));
    if (i == 0 && row < rows) {
      float res[1] = {C::apply(init, acc)};
      out[row] = Post::apply(res, caps.c + 8);
    }
  }
}

// Reduce over the INNERMOST axis of rows of at most 16 vectors with ONE THREAD PER ROW folding it in ascending
// order -- the order of the reference's SeqReducer (runtime/tca/reducer.h:45-51), which the reference's own suite
// tolerances (1e-5 absolute on sums of magnitude 32) in effect demand -- but with coalesced loads: a warp owns 32
// consecutive rows, which are one contiguous piece of memory; its lanes copy that piece vector by vector into
// shared memory (cp.async, 16 bytes per fp32 vector, 8 per bf16 vector, rows padded by one slot so that the 32
// lanes later read 32 different banks groups), and lane r then folds row r from there. chain_inner with a thread
// per row reads the same bytes with every load instruction touching 32 different rows.
// Dynamic shared memory: warps * NIN * 32 * (nvec + 1) * 16 bytes; blockDim.x = 32 * warps.
template <class Map, class Post, int COMBINE, int NIN, int BF = 0>
__global__ void __launch_bounds__(256)
chain_inner_rows32(Ptrs<NIN> ins, float* __restrict__ out, u64 rows, u32 nvec, float init, Caps caps) {
  typedef Comb<COMBINE> C;
  extern __shared__ __align__(16) unsigned char rows32_smem[];
  const u32 lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  const u64 row_base = (static_cast<u64>(blockIdx.x) * warps + warp) * 32;
  if (row_base >= rows) return;  // the whole warp leaves
  const u32 nrows = rows - row_base < 32 ? static_cast<u32>(rows - row_base) : 32u;
  const u32 pitch = nvec + 1;
  unsigned char* area = rows32_smem + static_cast<size_t>(warp) * NIN * 32 * pitch * 16;
  const u32 total = nrows * nvec;
  for (u32 v = lane; v < total; v += 32) {
    const u32 r = v / nvec, j = v - r * nvec;
#pragma unroll
    for (int a = 0; a < NIN; ++a) {
      const unsigned dst = static_cast<unsigned>(__cvta_generic_to_shared(area + (static_cast<size_t>(a * 32 + r) * pitch + j) * 16));
      if ((BF >> a) & 1) {
        const unsigned char* src = reinterpret_cast<const unsigned char*>(ins.p[a]) + (row_base * nvec + v) * 8;
        asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst), "l"(src) : "memory");
      } else {
        const unsigned char* src = reinterpret_cast<const unsigned char*>(ins.p[a]) + (row_base * nvec + v) * 16;
        asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
      }
    }
  }
  asm volatile("cp.async.wait_all;" ::: "memory");
  __syncwarp();
  if (lane < nrows) {
    float acc = C::identity();
    for (u32 j = 0; j < nvec; ++j) {
      float f[NIN][4];
#pragma unroll
      for (int a = 0; a < NIN; ++a) {
        const unsigned char* slot = area + (static_cast<size_t>(a * 32 + lane) * pitch + j) * 16;
        if ((BF >> a) & 1) {
          const uint2 q = *reinterpret_cast<const uint2*>(slot);
          f[a][0] = bf16_bits_to_float(q.x & 0xffffu); f[a][1] = bf16_bits_to_float(q.x >> 16);
          f[a][2] = bf16_bits_to_float(q.y & 0xffffu); f[a][3] = bf16_bits_to_float(q.y >> 16);
        } else {
          const float4 q = *reinterpret_cast<const float4*>(slot);
          f[a][0] = q.x; f[a][1] = q.y; f[a][2] = q.z; f[a][3] = q.w;
        }
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float p[NIN];
#pragma unroll
        for (int a = 0; a < NIN; ++a) p[a] = f[a][e];
        acc = C::apply(acc, Map::apply(p, caps.c));
      }
    }
    float res[1] = {C::apply(init, acc)};
    out[row_base + lane] = Post::apply(res, caps.c + 8);
  }
}

// The same for short rows that are not whole vectors (nk % 4 != 0, aligned operands, nk <= 64): the 32 rows of a warp
// start at element 32 m nk -- a 128-byte boundary -- and are 8 nk whole vectors, whatever nk is, so the warp copies
// them as they lie (cp.async, 16 bytes; the last, shorter group of rows ends with up to three single elements) and
// lane r folds elements r nk ... r nk + nk - 1 of the copy in ascending order. Rows of an odd length fall on
// different banks; nk = 2 (mod 4) costs two-way conflicts.
// Dynamic shared memory: warps * NIN * 32 * nk * 4 bytes; blockDim.x = 32 * warps.
template <class Map, class Post, int COMBINE, int NIN, int BF = 0>
__global__ void __launch_bounds__(256)
chain_inner_rows32e(Ptrs<NIN> ins, float* __restrict__ out, u64 rows, u32 nk, float init, Caps caps) {
  typedef Comb<COMBINE> C;
  extern __shared__ __align__(16) unsigned char rows32_smem[];
  const u32 lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  const u64 row_base = (static_cast<u64>(blockIdx.x) * warps + warp) * 32;
  if (row_base >= rows) return;  // the whole warp leaves
  const u32 nrows = rows - row_base < 32 ? static_cast<u32>(rows - row_base) : 32u;
  unsigned char* area = rows32_smem + static_cast<size_t>(warp) * NIN * 32 * nk * 4;
  const u32 total = nrows * nk, nvec = total >> 2;
  const u64 e0 = row_base * nk;  // a multiple of 32 elements
  for (u32 v = lane; v < nvec; v += 32) {
#pragma unroll
    for (int a = 0; a < NIN; ++a) {
      unsigned char* slab = area + static_cast<size_t>(a) * 32 * nk * 4;
      if ((BF >> a) & 1) {
        const unsigned dst = static_cast<unsigned>(__cvta_generic_to_shared(slab + static_cast<size_t>(v) * 8));
        const unsigned char* src = reinterpret_cast<const unsigned char*>(ins.p[a]) + (e0 + 4ull * v) * 2;
        asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst), "l"(src) : "memory");
      } else {
        const unsigned dst = static_cast<unsigned>(__cvta_generic_to_shared(slab + static_cast<size_t>(v) * 16));
        const unsigned char* src = reinterpret_cast<const unsigned char*>(ins.p[a]) + (e0 + 4ull * v) * 4;
        asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
      }
    }
  }
  if (lane < (total & 3u)) {  // the end of the last group of rows
    const u32 e = 4 * nvec + lane;
#pragma unroll
    for (int a = 0; a < NIN; ++a) {
      unsigned char* slab = area + static_cast<size_t>(a) * 32 * nk * 4;
      if ((BF >> a) & 1) {
        reinterpret_cast<unsigned short*>(slab)[e] = reinterpret_cast<const unsigned short*>(ins.p[a])[e0 + e];
      } else {
        reinterpret_cast<float*>(slab)[e] = ins.p[a][e0 + e];
      }
    }
  }
  asm volatile("cp.async.wait_all;" ::: "memory");
  __syncwarp();
  if (lane < nrows) {
    float acc = C::identity();
    const u32 first = lane * nk;
    for (u32 j = 0; j < nk; ++j) {
      float p[NIN];
#pragma unroll
      for (int a = 0; a < NIN; ++a) {
        const unsigned char* slab = area + static_cast<size_t>(a) * 32 * nk * 4;
        if ((BF >> a) & 1) {
          p[a] = bf16_bits_to_float(reinterpret_cast<const unsigned short*>(slab)[first + j]);
        } else {
          p[a] = reinterpret_cast<const float*>(slab)[first + j];
        }
      }
      acc = C::apply(acc, Map::apply(p, caps.c));
    }
    float res[1] = {C::apply(init, acc)};
    out[row_base + lane] = Post::apply(res, caps.c + 8);
  }
}

// Several problems of ONE shape in one launch: problem b has operands ins.in[b][*] of [rows, nk] and output
// ins.out[b] of [rows]. A lone small reduction is bounded by what a launch costs and by the wait for its
// predecessor on the stream, not by memory (a [4096, 1024] fp32 input is 2.6 us of HBM time; a dependent launch
// adds more than a microsecond to it); a host that has many of them hands them over together, and the rows
// of all problems are one pool of work for the grid. The reference's launcher takes one problem per call
// (internal/cg/cxx/launch.go:23-156).
constexpr int kMaxBatch = 32;
template <int NIN>
struct BatchPtrs {
  const float* in[kMaxBatch][NIN];
  float* out[kMaxBatch];
};

template <class Map, class Post, int COMBINE, int NIN, int TPR, int V, int BF = 0>
__global__ void __launch_bounds__(256)
chain_inner_batched(BatchPtrs<NIN> ins, u32 nprob, u32 rows, u32 nk, float init, Caps caps) {
  typedef Comb<COMBINE> C;
  constexpr int GROUPS = 256 / TPR;
  __shared__ float slots[2][32];
  const int g = threadIdx.x / TPR;
  const int t = threadIdx.x % TPR;
  const u32 nvec = nk / V;
  const u64 total = static_cast<u64>(nprob) * rows;
  u32 iter = 0;
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  for (u64 row0 = static_cast<u64>(blockIdx.x) * GROUPS; row0 < total; row0 += static_cast<u64>(gridDim.x) * GROUPS, ++iter) {
    const u64 gr = row0 + g;
    const bool live = gr < total;
    const u32 b = live ? static_cast<u32>(gr / rows) : 0u;
    const u64 row = live ? gr % rows : 0;
    float acc = C::identity();
    if (live) acc = fold_row_share<Map, C, NIN, TPR, V, BF>(ins.in[b], row, nvec, t, caps.c);
    acc = fold_row_group<C, TPR>(acc, slots, iter);
    if (live && t == 0) {
      float r[1] = {C::apply(init, acc)};
      ins.out[b][row] = Post::apply(r, caps.c + 8);
    }
  }
}

// A long row split over several CTAs (the multi-CTA reduction the reference stubs as
// GlobalReducer, runtime/tca/reducer.h:187-213). Pass 1: CTA (row, s) folds vectors
// [s*vec_per_split, (s+1)*vec_per_split) of its row and writes ONE partial to
// partials[row*splits + s] (global scratch memory). Pass 2 (chain_split_finish) folds the
// partials of a row in ascending order, applies init and the piped map.
template <class Map, int COMBINE, int NIN, int V, int BF = 0>
__global__ void __launch_bounds__(256)
chain_inner_split(Ptrs<NIN> ins, float* __restrict__ partials, u32 nk, u32 splits, u32 vec_per_split, Caps caps) {
  typedef Comb<COMBINE> C;
  __shared__ float slots[8];
  const u32 row = blockIdx.x / splits, s = blockIdx.x % splits;
  const u32 nvec = nk / V;
  const u64 vbase = static_cast<u64>(row) * nvec;
  const u32 v0 = s * vec_per_split;
  const u32 v1 = (nvec - v0 < vec_per_split) ? nvec : v0 + vec_per_split;
  float acc = C::identity();
  if (v0 < nvec) {
#pragma unroll(V == 1 ? 16 : 4)  // 4-byte loads need more of them in flight for the same bytes
    for (u32 idx = v0 + threadIdx.x; idx < v1; idx += 256) {
      float f[NIN][V];
      LoadAll<V, BF, NIN>::at(ins.p, vbase + idx, f);
#pragma unroll
      for (int j = 0; j < V; ++j) {
        float p[NIN];
#pragma unroll
        for (int a = 0; a < NIN; ++a) p[a] = f[a][j];
        acc = C::apply(acc, Map::apply(p, caps.c));
      }
    }
  }
  acc = lanes_allreduce<C, 32>(acc);
  if ((threadIdx.x & 31) == 0) slots[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    acc = lanes_allreduce<C, 8>(slots[threadIdx.x & 7]);
    if (threadIdx.x == 0) partials[blockIdx.x] = acc;
  }
}

// `lanes` (a power of two up to 32) threads share a row's partials: 1 folds them in ascending order starting from init;
// more (many partials of few rows: the k ranges of a middle-axis reduction) take every lanes-th partial each and meet
// by shuffles, init joining last.
template <class Post, int COMBINE>
__global__ void __launch_bounds__(128)
chain_split_finish(const float* __restrict__ partials, float* __restrict__ out, u32 rows, u32 splits, float init,
                   Caps caps, u32 lanes) {
  typedef Comb<COMBINE> C;
  const u32 t = blockIdx.x * 128 + threadIdx.x;
  const u32 row = t / lanes, l = t % lanes;
  float a = lanes == 1 ? init : C::identity();
  if (row < rows) {
#pragma unroll 4
    for (u32 s = l; s < splits; s += lanes) a = C::apply(a, partials[static_cast<u64>(row) * splits + s]);
  }
  if (lanes > 1) {
    for (u32 off = lanes >> 1; off > 0; off >>= 1) a = C::apply(a, __shfl_xor_sync(0xffffffffu, a, off));
    a = C::apply(init, a);
  }
  if (row < rows && l == 0) {
    float r[1] = {a};
    out[row] = Post::apply(r, caps.c + 8);
  }
}

// Reduce over a MIDDLE axis: operands are [nb, nk, nc]; a CTA owns (one b, a
// tile of 32*V columns), lane l owns V columns, warp w owns k = w, w+KW, ...
// With ksplit > 1 the k axis is also cut into ksplit ranges of klen, one CTA each (few columns, long k):
// a CTA then writes the fold of its range -- without init and without the piped map -- to
// partials[cell * ksplit + range], and chain_split_finish folds the ranges in ascending order.
template <class Map, class Post, int COMBINE, int NIN, int V, int KW, int UNROLL, int BF = 0, int CELL = 0>
__global__ void __launch_bounds__(32 * KW)
chain_outer(Ptrs<NIN> ins, float* __restrict__ out, u32 nb, u32 nk, u32 nc, u32 tiles_per_b, float init,
            Caps caps, u32 ksplit, u32 klen, float* __restrict__ partials) {
  typedef Comb<COMBINE> C;
  constexpr int TILE_C = 32 * V;
  __shared__ float s_part[KW][TILE_C];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

  for (u32 work = blockIdx.x; work < nb * tiles_per_b * ksplit; work += gridDim.x) {
    const u32 tile = work / ksplit, ks = work % ksplit;
    // a range that would start past the end is empty (kbeg == kend) and contributes the combiner's identity
    const u32 kbeg = ks * klen < nk ? ks * klen : nk, kend = (nk - kbeg < klen) ? nk : kbeg + klen;
    const u32 b = tile / tiles_per_b;
    const u32 c0 = (tile % tiles_per_b) * TILE_C;
    const u32 col = c0 + lane * V;
    const bool colok = col < nc;  // nc % V == 0 when V == 4
    const u64 base = static_cast<u64>(b) * nk * nc + col;

    float acc[V];
#pragma unroll
    for (int j = 0; j < V; ++j) acc[j] = C::identity();

    if (colok) {
      float cellval[NIN][V];  // operands that lack the reduced axis: one value per output cell, loaded once
      LoadOuterAll<V, BF, CELL, NIN>::cells(ins.p, (static_cast<u64>(b) * nc + col) / V, cellval);
      for (u32 k0 = kbeg + warp; k0 < kend; k0 += KW * UNROLL) {
        float f[UNROLL][NIN][V];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
          const u32 k = k0 + u * KW;
          if (k < kend)  // base and k * nc are multiples of V on the vector path
            LoadOuterAll<V, BF, CELL, NIN>::at(ins.p, (base + static_cast<u64>(k) * nc) / V, cellval, f[u]);
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
          const u32 k = k0 + u * KW;
          if (k < kend) {
#pragma unroll
            for (int j = 0; j < V; ++j) {
              float p[NIN];
#pragma unroll
              for (int a = 0; a < NIN; ++a) p[a] = f[u][a][j];
              acc[j] = C::apply(acc[j], Map::apply(p, caps.c));
            }
          }
        }
      }
    }
#pragma unroll
    for (int j = 0; j < V; ++j) s_part[warp][lane * V + j] = acc[j];
    __syncthreads();
    for (int c = threadIdx.x; c < TILE_C; c += 32 * KW) {
      if (c0 + c < nc) {
        float a = ksplit > 1 ? C::identity() : init;
#pragma unroll
        for (int w = 0; w < KW; ++w) a = C::apply(a, s_part[w][c]);
        const u64 cell = static_cast<u64>(b) * nc + c0 + c;
        if (ksplit > 1) {
          partials[cell * ksplit + ks] = a;
        } else {
          float r[1] = {a};
          out[cell] = Post::apply(r, caps.c + 8);
        }
      }
    }
    __syncthreads();
  }
}

// Reduce over a MIDDLE axis with a WARP per (b, column tile), for the shapes on which chain_outer idles: narrow
// rows (most lanes of a CTA's column tile would have no column) and short reduced axes (a CTA per tile would do a
// few hundred bytes of work between two barriers). A lane loads V columns at once (V = 4: 16-byte vectors, nc % 4
// == 0 and aligned operands; V = 1: any nc, any alignment). The warp's lanes cover g column groups of V and 32 / g
// consecutive k rows per step (lanes beyond g * (32 / g) idle when g does not divide 32); when the tile is the whole
// row (nc = V g < 32 V) what a step loads is contiguous in memory. Every lane folds the k rows it sees (ascending),
// lanes with the same column group then meet by shuffles, and lanes 0..g-1 store. No shared memory, no barrier;
// eight independent warps per CTA.
template <class Map, class Post, int COMBINE, int NIN, int UNROLL, int BF = 0, int CELL = 0, int V = 4>
__global__ void __launch_bounds__(256)
chain_outer_flat(Ptrs<NIN> ins, float* __restrict__ out, u32 nb, u32 nk, u32 nc, u32 tiles_per_b, u32 g, float init,
                 Caps caps, u32 ksplit, u32 klen, float* __restrict__ partials) {
  // ksplit > 1 (few tiles, a long reduced axis): a CTA takes range blockIdx % ksplit of klen rows of ONE (b, column
  // tile); its eight warps interleave step by step, so that the CTA streams one contiguous piece of memory, and it
  // writes the fold of its rows -- without init and without the piped map -- to partials[cell * ksplit + range] for
  // chain_split_finish.
  typedef Comb<COMBINE> C;
  const u32 lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  u64 work;
  u32 kbeg = 0, kend = nk, kstep = (32 / g) * UNROLL, ks = 0;
  if (ksplit > 1) {
    work = blockIdx.x / ksplit;
    ks = blockIdx.x % ksplit;
    const u32 first = ks * klen < nk ? ks * klen : nk;  // a range that would start past the end is empty
    kend = nk - first < klen ? nk : first + klen;
    kbeg = first + warp * kstep;
    if (kbeg > kend) kbeg = kend;
    kstep *= 8;
  } else {
    work = static_cast<u64>(blockIdx.x) * 8 + warp;
    if (work >= static_cast<u64>(nb) * tiles_per_b) return;  // the whole warp leaves
  }
  const u32 b = static_cast<u32>(work / tiles_per_b), tile = static_cast<u32>(work % tiles_per_b);
  const u32 rows_per_step = 32 / g;
  const u32 cg = lane % g, kr = lane / g;    // this lane's column group, and its row inside a step
  const u32 col = tile * (32 * V) + cg * V;  // g < 32 only when one tile is the whole row
  const bool colok = col < nc && kr < rows_per_step;
  const u64 rowvecs = nc / V;
  const u64 base = static_cast<u64>(b) * nk * rowvecs + col / V;

  float acc[V];
#pragma unroll
  for (int j = 0; j < V; ++j) acc[j] = C::identity();
  if (colok) {
    float cellval[NIN][V];  // operands that lack the reduced axis: one value per output cell, loaded once
    LoadOuterAll<V, BF, CELL, NIN>::cells(ins.p, (static_cast<u64>(b) * nc + col) / V, cellval);
    u32 k0 = kbeg + kr;
    const u64 ustride = static_cast<u64>(rows_per_step) * rowvecs;
    // iterations whose UNROLL rows all exist: no predicates
    for (; kend > (UNROLL - 1) * rows_per_step && k0 < kend - (UNROLL - 1) * rows_per_step; k0 += kstep) {
      float f[UNROLL][NIN][V];
      const u64 at = base + static_cast<u64>(k0) * rowvecs;
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) LoadOuterAll<V, BF, CELL, NIN>::at(ins.p, at + u * ustride, cellval, f[u]);
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
#pragma unroll
        for (int j = 0; j < V; ++j) {
          float p[NIN];
#pragma unroll
          for (int a = 0; a < NIN; ++a) p[a] = f[u][a][j];
          acc[j] = C::apply(acc[j], Map::apply(p, caps.c));
        }
      }
    }
    for (; k0 < kend; k0 += kstep) {  // the ragged end of this lane's rows
      float f[UNROLL][NIN][V];
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const u32 k = k0 + u * rows_per_step;
        if (k < kend) LoadOuterAll<V, BF, CELL, NIN>::at(ins.p, base + static_cast<u64>(k) * rowvecs, cellval, f[u]);
      }
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const u32 k = k0 + u * rows_per_step;
        if (k < kend) {
#pragma unroll
          for (int j = 0; j < V; ++j) {
            float p[NIN];
#pragma unroll
            for (int a = 0; a < NIN; ++a) p[a] = f[u][a][j];
            acc[j] = C::apply(acc[j], Map::apply(p, caps.c));
          }
        }
      }
    }
  }
  if ((g & (g - 1)) == 0) {
    for (u32 off = 16; off >= g; off >>= 1) {  // lanes that differ in the row bits hold the same column group
#pragma unroll
      for (int j = 0; j < V; ++j) acc[j] = C::apply(acc[j], __shfl_xor_sync(0xffffffffu, acc[j], off));
    }
  } else {  // lanes cg, cg + g, cg + 2 g, ... hold column group cg: lanes 0..g-1 collect them in row order
    for (u32 r = 1; r < rows_per_step; ++r) {
#pragma unroll
      for (int j = 0; j < V; ++j) {
        const float v = __shfl_sync(0xffffffffu, acc[j], (lane + r * g) & 31);
        if (lane < g) acc[j] = C::apply(acc[j], v);
      }
    }
  }
  if (ksplit > 1) {  // the CTA's warps meet in shared memory, in warp order: one partial per range and cell
    __shared__ float s_part[8][128];
    if (lane < g) {
#pragma unroll
      for (int j = 0; j < V; ++j) s_part[warp][cg * V + j] = acc[j];
    }
    __syncthreads();
    const u32 c = threadIdx.x, tile_col = tile * (32 * V) + c;
    if (c < V * g && tile_col < nc) {
      float a = s_part[0][c];
#pragma unroll
      for (int w = 1; w < 8; ++w) a = C::apply(a, s_part[w][c]);
      partials[(static_cast<u64>(b) * nc + tile_col) * ksplit + ks] = a;
    }
    return;
  }
  if (lane < g && colok) {
    const u64 cell = static_cast<u64>(b) * nc + col;
#pragma unroll
    for (int j = 0; j < V; ++j) {
      float r[1] = {C::apply(init, acc[j])};
      out[cell + j] = Post::apply(r, caps.c + 8);
    }
  }
}

// Contraction of two fp32 operands indexed by different dim subsets (the reference's matmul-shaped
// chains: testing/kernels/llm/gemm.tca, tiling/mm_*.tca, fusion/mlp.tca, llm/qk_score.tca):
//   out[m,n] = post( fold_k map(lhs[m,k], rhs[k,n]) )         RHS_NK == 0, rhs is [K,N]
//   out[m,n] = post( fold_k map(lhs[m,k], rhs[n,k]) )         RHS_NK == 1, rhs is [N,K]
// 256 threads own a (16 TM) x (16 TM) output tile, a thread TM x TM of it as 4x4 blocks 64 rows /
// columns apart (TM = 4: 64x64 tiles for small problems; TM = 8: 128x128 tiles). K advances in
// shared-memory tiles of 16, double-buffered: the next tile's global loads (16-byte vectors where the
// row pitch allows) are in registers while the current one is multiplied. Operands whose k runs fastest
// in memory are stored transposed, so that the inner loop reads 16-byte vectors along m and n (the row
// pitch of 16 TM + 4 floats keeps those vectors aligned and the transposing stores at two-way conflicts).
// Each output is folded over k in ascending order by one thread -- the order of the reference's CPU
// loops (testing/runners/gemm.cu:44-56). Rows and columns past the edge are computed on zero padding
// and never stored; k past the edge never reaches the lambda.
template <int TM>
struct ContractTile {
  static constexpr int BM = 16 * TM, BK = 16, PITCH = BM + 4;
  static constexpr int V = BM * BK / 4 / 256;  // 16-byte vectors per thread and operand tile (1 or 2)
};

// A [rows, K] operand (k fastest): vector v of the thread covers row r = idx / 4, k = (idx % 4) * 4 .. +3.
// Four consecutive elements at element offset `e` of an operand (fp32, or bf16 widened): one 16-byte
// (8-byte) load when the caller has checked alignment and bounds, else up to `valid` single elements.
template <bool IS_BF16>
__device__ __forceinline__ void contract_load4(const float* __restrict__ p, u64 e, bool vec, int valid, float (&r)[4]) {
  if constexpr (IS_BF16) {
    const unsigned short* h = reinterpret_cast<const unsigned short*>(p) + e;
    if (vec) {
      const uint2 q = *reinterpret_cast<const uint2*>(h);
      r[0] = bf16_bits_to_float(q.x & 0xffffu); r[1] = bf16_bits_to_float(q.x >> 16);
      r[2] = bf16_bits_to_float(q.y & 0xffffu); r[3] = bf16_bits_to_float(q.y >> 16);
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) r[j] = j < valid ? bf16_bits_to_float(h[j]) : 0.0f;
    }
  } else {
    const float* src = p + e;
    if (vec) {
      const float4 q = *reinterpret_cast<const float4*>(src);
      r[0] = q.x; r[1] = q.y; r[2] = q.z; r[3] = q.w;
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) r[j] = j < valid ? src[j] : 0.0f;
    }
  }
}

template <int TM, bool IS_BF16>
__device__ __forceinline__ void contract_fetch_k_fastest(const float* __restrict__ p, u32 row0, u32 rows, u32 k0, u32 K,
                                                         bool vec_ok, float (&reg)[ContractTile<TM>::V][4]) {
#pragma unroll
  for (int v = 0; v < ContractTile<TM>::V; ++v) {
    const int idx = threadIdx.x + v * 256;
    const u32 r = row0 + (idx >> 2), k = k0 + (idx & 3) * 4;
    const int valid = r < rows && k < K ? static_cast<int>(K - k < 4u ? K - k : 4u) : 0;
    contract_load4<IS_BF16>(p, static_cast<u64>(r) * K + k, vec_ok && valid == 4, valid, reg[v]);
  }
}
template <int TM>
__device__ __forceinline__ void contract_stash_k_fastest(float (*tile)[ContractTile<TM>::PITCH],
                                                         const float (&reg)[ContractTile<TM>::V][4]) {
#pragma unroll
  for (int v = 0; v < ContractTile<TM>::V; ++v) {
    const int idx = threadIdx.x + v * 256;
    const int r = idx >> 2, k = (idx & 3) * 4;
#pragma unroll
    for (int j = 0; j < 4; ++j) tile[k + j][r] = reg[v][j];
  }
}
// B as [K, N] (n fastest): vector v covers k = idx / (BM / 4), n = (idx % (BM / 4)) * 4 .. +3.
template <int TM, bool IS_BF16>
__device__ __forceinline__ void contract_fetch_n_fastest(const float* __restrict__ p, u32 n0, u32 N, u32 k0, u32 K,
                                                         bool vec_ok, float (&reg)[ContractTile<TM>::V][4]) {
  constexpr int W = ContractTile<TM>::BM / 4;
#pragma unroll
  for (int v = 0; v < ContractTile<TM>::V; ++v) {
    const int idx = threadIdx.x + v * 256;
    const u32 k = k0 + idx / W, n = n0 + (idx % W) * 4;
    const int valid = k < K && n < N ? static_cast<int>(N - n < 4u ? N - n : 4u) : 0;
    contract_load4<IS_BF16>(p, static_cast<u64>(k) * N + n, vec_ok && valid == 4, valid, reg[v]);
  }
}
template <int TM>
__device__ __forceinline__ void contract_stash_n_fastest(float (*tile)[ContractTile<TM>::PITCH],
                                                         const float (&reg)[ContractTile<TM>::V][4]) {
  constexpr int W = ContractTile<TM>::BM / 4;
#pragma unroll
  for (int v = 0; v < ContractTile<TM>::V; ++v) {
    const int idx = threadIdx.x + v * 256;
    *reinterpret_cast<float4*>(&tile[idx / W][(idx % W) * 4]) = make_float4(reg[v][0], reg[v][1], reg[v][2], reg[v][3]);
  }
}

template <class Map, class Post, int COMBINE, int RHS_NK, int TM, int BF = 0>
__global__ void __launch_bounds__(256, 2)
chain_contract(const float* __restrict__ lhs, const float* __restrict__ rhs, float* __restrict__ out, u32 M, u32 N,
               u32 K, float init, Caps caps) {
  typedef Comb<COMBINE> C;
  typedef ContractTile<TM> T;
  constexpr int BM = T::BM, BK = T::BK, Q = TM / 4;
  __shared__ __align__(16) float As[2][BK][T::PITCH];
  __shared__ __align__(16) float Bs[2][BK][T::PITCH];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const u32 m0 = blockIdx.y * BM, n0 = blockIdx.x * BM;
  const bool a_vec = (K % 4 == 0) && (reinterpret_cast<unsigned long long>(lhs) % 16 == 0);
  const bool b_vec = ((RHS_NK ? K : N) % 4 == 0) && (reinterpret_cast<unsigned long long>(rhs) % 16 == 0);
  float acc[TM][TM];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TM; ++j) acc[i][j] = C::identity();

  constexpr bool ABF = (BF & 1) != 0, BBF = (BF & 2) != 0;  // bf16 operands are widened to f32 at the load
  float ra[T::V][4], rb[T::V][4];
  if (K > 0) {
    contract_fetch_k_fastest<TM, ABF>(lhs, m0, M, 0, K, a_vec, ra);
    if (RHS_NK) contract_fetch_k_fastest<TM, BBF>(rhs, n0, N, 0, K, b_vec, rb);
    else contract_fetch_n_fastest<TM, BBF>(rhs, n0, N, 0, K, b_vec, rb);
    contract_stash_k_fastest<TM>(As[0], ra);
    if (RHS_NK) contract_stash_k_fastest<TM>(Bs[0], rb);
    else contract_stash_n_fastest<TM>(Bs[0], rb);
  }
  __syncthreads();

  int cur = 0;
  for (u32 k0 = 0; k0 < K; k0 += BK, cur ^= 1) {
    const bool more = k0 + BK < K;
    if (more) {  // the next tile travels while this one is multiplied
      contract_fetch_k_fastest<TM, ABF>(lhs, m0, M, k0 + BK, K, a_vec, ra);
      if (RHS_NK) contract_fetch_k_fastest<TM, BBF>(rhs, n0, N, k0 + BK, K, b_vec, rb);
      else contract_fetch_n_fastest<TM, BBF>(rhs, n0, N, k0 + BK, K, b_vec, rb);
    }
    const int kmax = (K - k0 < static_cast<u32>(BK)) ? static_cast<int>(K - k0) : BK;
    auto step = [&](int kk) {
      float a[TM], b[TM];
#pragma unroll
      for (int q = 0; q < Q; ++q) {
        const float4 va = *reinterpret_cast<const float4*>(&As[cur][kk][q * 64 + ty * 4]);
        const float4 vb = *reinterpret_cast<const float4*>(&Bs[cur][kk][q * 64 + tx * 4]);
        a[q * 4] = va.x; a[q * 4 + 1] = va.y; a[q * 4 + 2] = va.z; a[q * 4 + 3] = va.w;
        b[q * 4] = vb.x; b[q * 4 + 1] = vb.y; b[q * 4 + 2] = vb.z; b[q * 4 + 3] = vb.w;
      }
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TM; ++j) {
          const float p[2] = {a[i], b[j]};
          acc[i][j] = C::apply(acc[i][j], Map::apply(p, caps.c));
        }
    };
    if (kmax == BK) {
#pragma unroll
      for (int kk = 0; kk < BK; ++kk) step(kk);
    } else {
      for (int kk = 0; kk < kmax; ++kk) step(kk);
    }
    if (more) {
      contract_stash_k_fastest<TM>(As[cur ^ 1], ra);
      if (RHS_NK) contract_stash_k_fastest<TM>(Bs[cur ^ 1], rb);
      else contract_stash_n_fastest<TM>(Bs[cur ^ 1], rb);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const u32 m = m0 + (i / 4) * 64 + ty * 4 + (i % 4);
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < TM; ++j) {
      const u32 n = n0 + (j / 4) * 64 + tx * 4 + (j % 4);
      if (n >= N) continue;
      const float r[1] = {C::apply(init, acc[i][j])};
      out[static_cast<u64>(m) * N + n] = Post::apply(r, caps.c + 8);
    }
  }
}

// ---------------------------------------------------------------------------------------------------
// Map-only chain with a rank-preserving store: out[i] = map(ins[0][i], ins[1][i], ...) over n elements of
// identically shaped operands. The reference's rungs cannot store a map without a reduction
// (pkg/chain.go:433-438); its emitted code for a map statement is one predicated TensorView::Get per operand
// and one Set per element (runtime/tca/view.h:104-112). Here a thread owns EPT = 8 consecutive elements: per
// operand two 16-byte loads (f32 / i32 / u32) or one (bf16), all issued before the first lambda, and the same
// on the store side. The last n % 8 elements are done one by one by the thread after the last full group.
// EPT = 1 is the same kernel with single-element accesses, for pointers that are not 16-byte aligned.
// OUT_BF16: the result is rounded to bf16 (the functor returns the bf16 value widened to f32, exactly).
template <int EPT, bool IS_BF16>
struct MapLd;
template <>
struct MapLd<8, false> {
  static __device__ __forceinline__ void load(const float* base, u64 group, float* f) {
    const float4 a = __ldcs(reinterpret_cast<const float4*>(base) + 2 * group);
    const float4 b = __ldcs(reinterpret_cast<const float4*>(base) + 2 * group + 1);
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
  }
};
template <>
struct MapLd<8, true> {
  static __device__ __forceinline__ void load(const float* base, u64 group, float* f) {
    const uint4 q = __ldcs(reinterpret_cast<const uint4*>(base) + group);
    const unsigned int w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      f[2 * i] = bf16_bits_to_float(w[i] & 0xffffu);
      f[2 * i + 1] = bf16_bits_to_float(w[i] >> 16);
    }
  }
};
template <>
struct MapLd<1, false> {
  static __device__ __forceinline__ void load(const float* base, u64 i, float* f) { f[0] = __ldcs(base + i); }
};
template <>
struct MapLd<1, true> {
  static __device__ __forceinline__ void load(const float* base, u64 i, float* f) {
    f[0] = bf16_bits_to_float(__ldcs(reinterpret_cast<const unsigned short*>(base) + i));
  }
};
// index: the group (EPT = 8) or element (EPT = 1) in the flat output; row / col_index: the same position as a
// row and a group or element within the row, for operands with one value per row (RB) or one shared row (CB).
template <int EPT, int BF, int RB, int CB, int NIN, int A = 0>
struct MapLoadAll {
  static __device__ __forceinline__ void at(const float* const* p, u64 index, u64 row, u64 col_index, float (*f)[EPT]) {
    constexpr bool bf = ((BF >> A) & 1) != 0;
    if constexpr (((RB >> A) & 1) != 0) {
      float v;
      MapLd<1, bf>::load(p[A], row, &v);
#pragma unroll
      for (int j = 0; j < EPT; ++j) f[A][j] = v;
    } else if constexpr (((CB >> A) & 1) != 0) {
      MapLd<EPT, bf>::load(p[A], col_index, f[A]);
    } else {
      MapLd<EPT, bf>::load(p[A], index, f[A]);
    }
    MapLoadAll<EPT, BF, RB, CB, NIN, A + 1>::at(p, index, row, col_index, f);
  }
};
template <int EPT, int BF, int RB, int CB, int NIN>
struct MapLoadAll<EPT, BF, RB, CB, NIN, NIN> {
  static __device__ __forceinline__ void at(const float* const*, u64, u64, u64, float (*)[EPT]) {}
};

// The same for a group of eight that may straddle rows (cols % 8 != 0): operands of the full shape still load
// their 32 (16) aligned bytes; an operand with one value per row or one shared row is read element by element, the
// (row, column) of the group's first element advanced without further divisions.
template <int BF, int RB, int CB, int NIN, int A = 0>
struct MapLoadRagged {
  static __device__ __forceinline__ void at(const float* const* p, u64 group, u64 row0, u32 col0, u32 cols, float (*f)[8]) {
    constexpr bool bf = ((BF >> A) & 1) != 0;
    if constexpr ((((RB | CB) >> A) & 1) != 0) {
      u64 row = row0;
      u32 col = col0;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (col >= cols) {  // cols >= 1: at most one row ends per element
          col = 0;
          ++row;
        }
        MapLd<1, bf>::load(p[A], ((RB >> A) & 1) ? row : static_cast<u64>(col), &f[A][j]);
        ++col;
      }
    } else {
      MapLd<8, bf>::load(p[A], group, f[A]);
    }
    MapLoadRagged<BF, RB, CB, NIN, A + 1>::at(p, group, row0, col0, cols, f);
  }
};
template <int BF, int RB, int CB, int NIN>
struct MapLoadRagged<BF, RB, CB, NIN, NIN> {
  static __device__ __forceinline__ void at(const float* const*, u64, u64, u32, u32, float (*)[8]) {}
};

template <int NIN, int BF, int RB, int CB, bool OUT_BF16, class Map>
__device__ __forceinline__ void map_one(const float* const* p, void* out, u64 i, u32 cols, const float* caps) {
  float f[NIN][1];
  MapLoadAll<1, BF, RB, CB, NIN>::at(p, i, (RB | CB) ? i / cols : 0, (RB | CB) ? i % cols : 0, f);
  float v[NIN];
#pragma unroll
  for (int a = 0; a < NIN; ++a) v[a] = f[a][0];
  const float r = Map::apply(v, caps);
  if constexpr (OUT_BF16) static_cast<unsigned short*>(out)[i] = static_cast<unsigned short>(float_to_bf16_bits(r));
  else __stcs(static_cast<float*>(out) + i, r);
}

// One group of eight elements of a map: the operands' loads ...
template <int NIN, int BF, int RB, int CB>
__device__ __forceinline__ void map_load_group(const float* const* p, u64 group, u32 cols, float (*f)[8]) {
  if ((RB | CB) != 0 && cols % 8 != 0) {        // a group may straddle rows
    const u32 first = static_cast<u32>(group) * 8, row0 = first / cols;  // element counts are below 2^32
    MapLoadRagged<BF, RB, CB, NIN>::at(p, group, row0, first - row0 * cols, cols, f);
  } else {
    // groups per row; element counts are below 2^32 (the entry points refuse more), so 32-bit division will do
    const u32 gpr = (RB | CB) ? cols / 8 : 1, t32 = static_cast<u32>(group), row = (RB | CB) ? t32 / gpr : 0;
    MapLoadAll<8, BF, RB, CB, NIN>::at(p, group, row, (RB | CB) ? t32 - row * gpr : 0, f);
  }
}
// ... and the lambda on them with the store of its results.
template <class Map, int NIN, bool OUT_BF16>
__device__ __forceinline__ void map_apply_group(const float (*f)[8], void* out, u64 group, const float* caps) {
  float r[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    float v[NIN];
#pragma unroll
    for (int a = 0; a < NIN; ++a) v[a] = f[a][j];
    r[j] = Map::apply(v, caps);
  }
  if constexpr (OUT_BF16) {
    uint4 q;
    q.x = pack_bf16x2(r[0], r[1]);
    q.y = pack_bf16x2(r[2], r[3]);
    q.z = pack_bf16x2(r[4], r[5]);
    q.w = pack_bf16x2(r[6], r[7]);
    __stcs(static_cast<uint4*>(out) + group, q);
  } else {
    __stcs(static_cast<float4*>(out) + 2 * group, make_float4(r[0], r[1], r[2], r[3]));
    __stcs(static_cast<float4*>(out) + 2 * group + 1, make_float4(r[4], r[5], r[6], r[7]));
  }
}

// cols: the innermost extent; only read when an operand is broadcast (RB | CB != 0). A group of eight that
// straddles rows (cols % 8 != 0) reads its broadcast operands element by element. GPT: groups per thread, 256 apart
// (a CTA covers 256 GPT consecutive groups), the loads of all of them issued before the first lambda runs. Every
// launcher uses one: two were measured for maps over bf16 operands, whose group is 16 bytes per operand where an f32
// group is 32, and were slower (bias + ReLU on bf16 4.1 -> 3.6 TB/s: those maps are bound by instructions).
template <class Map, int NIN, int BF, bool OUT_BF16, int EPT, int RB = 0, int CB = 0, int GPT = 1>
__global__ void __launch_bounds__(256)
chain_map(Ptrs<NIN> ins, void* __restrict__ out, u64 n, Caps caps, u32 cols) {
  if constexpr (EPT == 1) {
    const u64 tid = static_cast<u64>(blockIdx.x) * 256 + threadIdx.x;
    if (tid < n) map_one<NIN, BF, RB, CB, OUT_BF16, Map>(ins.p, out, tid, cols, caps.c);
  } else {
    const u64 groups = n / 8;
    const u64 first = static_cast<u64>(blockIdx.x) * (256 * GPT) + threadIdx.x;
    float f[GPT][NIN][8];
#pragma unroll
    for (int q = 0; q < GPT; ++q)
      if (first + q * 256 < groups) map_load_group<NIN, BF, RB, CB>(ins.p, first + q * 256, cols, f[q]);
#pragma unroll
    for (int q = 0; q < GPT; ++q) {
      const u64 g = first + q * 256;
      if (g < groups) {
        map_apply_group<Map, NIN, OUT_BF16>(f[q], out, g, caps.c);
      } else if (g == groups) {  // the ragged end, fewer than eight elements
        for (u64 i = groups * 8; i < n; ++i) map_one<NIN, BF, RB, CB, OUT_BF16, Map>(ins.p, out, i, cols, caps.c);
      }
    }
  }
}

}  // namespace tcabk
