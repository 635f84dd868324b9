// rowvec.cuh -- element/vector adaptors and launch-shape choice for the row kernels
// (softmax, layer-norm, innermost-axis chains).
//
// A row is processed by a GROUP of TPR threads; thread t of the group owns the
// vectors t, t+TPR, t+2*TPR, ... of the row, so that one load instruction of a
// warp covers 32 consecutive 16-byte vectors (512 contiguous bytes). The
// reference's views read one bounds-checked scalar per access
// (runtime/tca/view.h:104-112); here the bounds test is one compare per vector.
#pragma once

#include "common.cuh"

namespace tcab {

#ifdef __CUDACC__

// VecIO<T, V>: V elements of type T moved as one access, unpacked to fp32.
template <typename T, int V>
struct VecIO;

template <>
struct VecIO<float, 4> {
  using Raw = float4;
  static __device__ __forceinline__ Raw load(const float* row, uint32_t i) {
    return ld_stream(reinterpret_cast<const float4*>(row) + i);
  }
  static __device__ __forceinline__ Raw load_keep(const float* row, uint32_t i) {
    return __ldg(reinterpret_cast<const float4*>(row) + i);
  }
  static __device__ __forceinline__ void store(float* row, uint32_t i, Raw r) {
    st_stream(reinterpret_cast<float4*>(row) + i, r);
  }
  static __device__ __forceinline__ void unpack(Raw r, float* f) {
    f[0] = r.x; f[1] = r.y; f[2] = r.z; f[3] = r.w;
  }
  static __device__ __forceinline__ Raw pack(const float* f) { return make_float4(f[0], f[1], f[2], f[3]); }
};

template <>
struct VecIO<float, 1> {
  using Raw = float;
  static __device__ __forceinline__ Raw load(const float* row, uint32_t i) { return ld_stream(row + i); }
  static __device__ __forceinline__ Raw load_keep(const float* row, uint32_t i) { return __ldg(row + i); }
  static __device__ __forceinline__ void store(float* row, uint32_t i, Raw r) { st_stream(row + i, r); }
  static __device__ __forceinline__ void unpack(Raw r, float* f) { f[0] = r; }
  static __device__ __forceinline__ Raw pack(const float* f) { return f[0]; }
};

// bf16 is a storage type: widened to fp32 on load, rounded to nearest even on
// store (design/syntax-design.md:601-607).
template <>
struct VecIO<__nv_bfloat16, 8> {
  using Raw = uint4;
  static __device__ __forceinline__ Raw load(const __nv_bfloat16* row, uint32_t i) {
    return ld_stream(reinterpret_cast<const uint4*>(row) + i);
  }
  static __device__ __forceinline__ Raw load_keep(const __nv_bfloat16* row, uint32_t i) {
    return __ldg(reinterpret_cast<const uint4*>(row) + i);
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* row, uint32_t i, Raw r) {
    st_stream(reinterpret_cast<uint4*>(row) + i, r);
  }
  static __device__ __forceinline__ void unpack(Raw r, float* f) {
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      f[2 * j] = __uint_as_float(w[j] << 16);
      f[2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
    }
  }
  static __device__ __forceinline__ Raw pack(const float* f) {
    uint32_t w[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * j], f[2 * j + 1]);
      w[j] = *reinterpret_cast<const uint32_t*>(&h);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
  }
};

template <>
struct VecIO<__nv_bfloat16, 1> {
  using Raw = __nv_bfloat16;
  static __device__ __forceinline__ Raw load(const __nv_bfloat16* row, uint32_t i) { return row[i]; }
  static __device__ __forceinline__ Raw load_keep(const __nv_bfloat16* row, uint32_t i) { return row[i]; }
  static __device__ __forceinline__ void store(__nv_bfloat16* row, uint32_t i, Raw r) { row[i] = r; }
  static __device__ __forceinline__ void unpack(Raw r, float* f) { f[0] = __bfloat162float(r); }
  static __device__ __forceinline__ Raw pack(const float* f) { return __float2bfloat16_rn(f[0]); }
};

// Reduction across the TPR threads of row group `g` of the CTA; every thread of the group gets
// the result. TPR <= 32: shuffles only. TPR > 32: the group's TPR/32 warps meet in `slots`
// (one float per warp of the CTA) behind ONE CTA-wide barrier, so every group of the CTA must
// call this the same number of times; the caller alternates between two slot arrays so that a
// slot is never rewritten before every thread has read it.
template <typename Op, int TPR>
__device__ __forceinline__ float group_allreduce(float v, float* slots, int g) {
  if constexpr (TPR <= 32) {
    return warp_allreduce<Op, TPR>(v);
  } else {
    constexpr int NW = TPR / 32;
    static_assert((NW & (NW - 1)) == 0 && NW <= 32, "a row group is a power-of-two number of warps");
    const int lane = threadIdx.x & 31, wg = (threadIdx.x % TPR) >> 5;
    v = warp_allreduce<Op>(v);
    if (lane == 0) slots[g * NW + wg] = v;
    __syncthreads();
    // every aligned group of NW lanes holds all the partials of the row group
    return warp_allreduce<Op, NW>(slots[g * NW + (lane & (NW - 1))]);
  }
}

#endif  // __CUDACC__

// CTA size of a row kernel whose groups have TPR threads: at least 128 threads,
// so that short rows still fill a CTA with several rows.
__host__ __device__ constexpr int row_cta_threads(int tpr) { return tpr > 128 ? tpr : 128; }

// Resident CTAs per SM to ask the compiler for. While a thread holds at most `limit` row values the
// kernel fits 48 registers, which lets 1280 threads (five 256-thread CTAs) share an SM instead of
// 1024: measured on B200, layer-norm over bf16 [65536, 8192] goes from 6.2 to 6.6 TB/s. Wider
// per-thread rows are left unconstrained (the cap would spill).
__host__ __device__ constexpr int row_min_ctas(int tpr, int values_per_thread, int limit, int threads_per_sm = 1280) {
  return values_per_thread <= limit && row_cta_threads(tpr) <= threads_per_sm ? threads_per_sm / row_cta_threads(tpr)
                                                                              : 1;
}

// Launch shape for a register-resident row: the smallest group (power of two,
// 8..1024 threads) whose threads hold at most `vpt_target` vectors each, and
// the power-of-two vector count per thread that then covers the row.
// Returns false when the row does not fit 1024 threads x 32 vectors.
inline bool choose_row_shape(uint32_t nvec, int vpt_target, int* tpr, int* vpt) {
  if (nvec == 0) nvec = 1;
  uint32_t t = pow2_ceil((nvec + vpt_target - 1) / vpt_target);
  if (t < 8) t = 8;
  if (t > 1024) t = 1024;
  uint32_t v = pow2_ceil((nvec + t - 1) / t);
  if (v > 32) return false;
  *tpr = static_cast<int>(t);
  *vpt = static_cast<int>(v);
  return true;
}

// The same choice with exact fits in mind. The row kernels skip vector slots that cannot hold data (a thread
// uses ceil(nvec / TPR) of its VPT slots), so what a shape wastes is only the idle threads of the last used
// slot: used * TPR / nvec. Among the compiled shapes -- (TPR, 4) for every power of two, (8, 1), (8, 2),
// (1024, 8..32) and, for 16-byte vectors, (128, 8), (256, 8), (64, 16), (32, 32) [plus (512, 8) and (64, 8)
// where `wide8`] -- this picks the least waste, preferring fewer slots and 128..512 threads on a tie, and
// staying at 32 row values per thread unless that wastes more than a third.
// `odd_slots`: the caller also has (16..256, 5) and (16..512, 3) -- rows of 5 * 2^k and 3 * 2^k vectors (hidden sizes
// 640, 768, 1280, 1536, 2560, 3072, 5120, 6144 ...) then fit exactly with every slot used (bf16 layer-norm, TB/s,
// best power-of-two shape -> exact fit: 1280 columns 5.1 -> 6.1, 5120 5.1 -> 5.9, 1536 5.7 -> 6.1, 3072 5.9 -> 6.3).
// fp32 rows gain from three slots everywhere but from five only with 32 threads per row (640 columns 6.4 -> 6.9; 64 x 5
// at 1280 columns 6.4 -> 6.2, 256 x 5 at 5120 columns 5.8 -> 5.0): `five_slots_max_threads`.
inline bool choose_row_shape_fit(uint32_t nvec, bool vec, bool wide8, int values_per_vector, int* tpr, int* vpt,
                                 bool small = false, double wide_penalty = 0.03, bool odd_slots = false,
                                 int five_slots_max_threads = 256) {
  if (nvec == 0) nvec = 1;
  struct Shape { int t, v; bool vec_only, wide_only, odd_only; };
  // rows of one to four vectors: one, two or four threads per row (`small`: the aligned register kernels have
  // these shapes; with eight threads per row a 4-column softmax ran at 0.95 TB/s, seven of eight threads idle)
  if (small && nvec <= 4) {
    *tpr = nvec <= 1 ? 1 : nvec <= 2 ? 2 : 4;
    *vpt = 1;
    return true;
  }
  static const Shape kShapes[] = {
      {8, 1, false, false},   {8, 2, false, false},    {8, 4, false, false},    {16, 4, false, false},
      {32, 4, false, false},  {64, 4, false, false},   {128, 4, false, false},  {256, 4, false, false},
      {512, 4, false, false}, {1024, 4, false, false}, {1024, 8, false, false}, {1024, 16, false, false},
      {1024, 32, false, false}, {128, 8, true, false}, {256, 8, true, false},   {64, 16, true, false},
      {32, 32, true, false},  {512, 8, true, true},    {64, 8, true, true},
      {16, 3, true, false, true},  {32, 3, true, false, true},  {64, 3, true, false, true}, {128, 3, true, false, true},
      {256, 3, true, false, true}, {512, 3, true, false, true}, {16, 5, true, false, true}, {32, 5, true, false, true},
      {64, 5, true, false, true},  {128, 5, true, false, true}, {256, 5, true, false, true}};
  double best = 1e30;
  bool found = false;
  for (const Shape& sh : kShapes) {
    if ((sh.vec_only && !vec) || (sh.wide_only && !wide8) || (sh.odd_only && !odd_slots)) continue;
    if (static_cast<uint64_t>(sh.t) * sh.v < nvec) continue;
    const uint32_t used = (nvec + sh.t - 1) / sh.t;
    if (sh.odd_only && used != static_cast<uint32_t>(sh.v)) continue;   // three or five slots only when all are used
    if (sh.odd_only && sh.v == 5 && sh.t > five_slots_max_threads) continue;
    double score = static_cast<double>(used) * sh.t / nvec;        // 1.0 = exact fit
    // more slots: more registers, fewer resident rows (five slots: a fifth of the penalty of eight)
    score *= 1.0 + wide_penalty * (sh.v > 4 ? (sh.v > 8 ? 2.0 : sh.v > 5 ? 1.0 : 0.2) : 0.0);
    score *= 1.0 + 0.02 * (sh.v - static_cast<int>(used));         // empty slots still cost their registers
    if (sh.v * values_per_vector > (odd_slots ? 40 : 32)) score *= 1.35;  // beyond that many row values per thread the kernels lose occupancy
    if (sh.t >= 1024) score *= 1.15;                               // 1024-thread CTAs move in lock step
    else if (sh.t < 16 && nvec > 32) score *= 1.10;                // short groups: strided 16-byte loads (16 threads x
                                                                   // 4 slots measured AHEAD of 32 x 2 on 64-vector rows:
                                                                   // bf16 layer-norm at 512 columns 6.6 against 4.9 TB/s)
    if (score < best - 1e-9) {
      best = score;
      *tpr = sh.t;
      *vpt = sh.v;
      found = true;
    }
  }
  return found;
}

// The register-row shape each operator asks for on aligned rows of nvec 16-byte vectors (the calls the dispatchers
// make, in one place so that a host without a device can sweep them): softmax (fp32), layer-norm fp32 / bf16.
inline bool softmax_row_shape(uint32_t nvec, bool vec, int* tpr, int* vpt) {
  return choose_row_shape_fit(nvec, vec, /*wide8=*/false, vec ? 4 : 1, tpr, vpt, /*small=*/true, /*wide_penalty=*/0.03,
                              /*odd_slots=*/vec, /*five_slots_max_threads=*/32);
}
inline bool layernorm_row_shape(uint32_t nvec, bool vec, int elem_bytes, int* tpr, int* vpt) {
  // fp32 rows: eight slots per thread (32 row values) cost resident rows; four slots on twice the threads measured
  // ahead even when a quarter of them idle (1280 columns 5.4 -> 6.2 TB/s, 5120 4.8 -> 5.7, 7168 5.7 -> 6.4)
  const int values_per_vector = vec ? 16 / elem_bytes : 1;
  return choose_row_shape_fit(nvec, vec, /*wide8=*/true, values_per_vector, tpr, vpt, /*small=*/true,
                              /*wide_penalty=*/elem_bytes == 4 ? 0.25 : 0.03, /*odd_slots=*/vec,
                              /*five_slots_max_threads=*/elem_bytes == 4 ? 32 : 256);
}

// Streaming clusters (softmax_rows_cluster_stream, layernorm_rows_cluster_stream): CTAs per row for a row of
// nvec vectors when a CTA takes per_step vectors per step. Four steps per CTA with the smallest cluster that allows
// it; where that leaves exactly-filled CTAs behind, a larger cluster that covers the row in at most three nearly
// full steps was measured faster for fp32 rows (`prefer_three`).
inline uint32_t stream_cluster_size(uint32_t nvec, uint32_t per_step, bool prefer_three) {
  auto steps = [&](uint32_t c) { return ((nvec + c - 1) / c + per_step - 1) / per_step; };
  uint32_t cs = (nvec + 4u * per_step - 1) / (4u * per_step);
  cs = cs < 2 ? 2u : cs > 8 ? 8u : cs;
  if (prefer_three && steps(cs) >= 4)
    for (uint32_t c = cs + 1; c <= 8 && c <= 2 * cs; ++c)
      if (steps(c) <= 3 && static_cast<uint64_t>(nvec) * 10 >= static_cast<uint64_t>(c) * steps(c) * per_step * 9) return c;
  return cs;
}

}  // namespace tcab
