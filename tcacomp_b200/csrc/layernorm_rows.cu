// layernorm_rows.cu -- layer-norm over the innermost axis as ONE fused
// map | reduce | map | reduce | map kernel with fp32 statistics.
//
//   mean = sum_j x / n;  var = sum_j (x - mean)^2 / n;
//   y = (x - mean) * (1 / sqrtf(var + eps)) * gamma + beta
//
// The reference's builder cannot express the rank-preserving store and ships an
// RMS-flavoured reduction core instead (testing/kernels/llm/layernorm.tca:1-40,
// runner testing/runners/layernorm.cu:47-58). bf16 rows are widened to fp32 on
// load and rounded to nearest even on store (design/syntax-design.md:601-607).
//
// The row lives in registers, so x is read once and y written once (4 bytes per
// bf16 element, 8 per fp32 element: the roofline figure). gamma and beta are either re-read per row through the read-only
// L1 path (they total a few KB and stay L1-resident; the row itself streams past
// L1), or, with CACHE_GB, kept in registers as raw 16-byte vectors across all the
// rows a thread processes. The first costs load-store issue slots, the second
// registers and therefore resident rows per SM; the launcher picks.
#include "rowvec.cuh"

namespace tcab {
namespace {

template <typename T, int TPR, int VPT, int V, bool CACHE_GB>
__global__ void __launch_bounds__(row_cta_threads(TPR), CACHE_GB ? 1 : row_min_ctas(TPR, VPT * V, sizeof(T) == 2 ? 32 : 16, TPR == 512 ? 1536 : TPR == 1024 ? 2048 : 1280))
layernorm_rows_reg(const T* __restrict__ x, const T* __restrict__ gamma, const T* __restrict__ beta,
                   float eps, T* __restrict__ y, uint64_t rows, uint32_t cols) {
  constexpr int THREADS = row_cta_threads(TPR);
  constexpr int GROUPS = THREADS / TPR;
  using IO = VecIO<T, V>;
  using Raw = typename IO::Raw;
  __shared__ float slots[2][32];

  const int g = threadIdx.x / TPR;
  const int t = threadIdx.x % TPR;
  const uint32_t nvec = cols / V;
  const float n = static_cast<float>(cols);

  Raw gv[CACHE_GB ? VPT : 1], bv[CACHE_GB ? VPT : 1];
#pragma unroll
  for (int i = 0; i < (CACHE_GB ? VPT : 0); ++i) {
    const uint32_t idx = t + i * TPR;
    if (idx < nvec) {
      gv[i] = IO::load_keep(gamma, idx);
      bv[i] = IO::load_keep(beta, idx);
    } else {
      float z[V];
#pragma unroll
      for (int j = 0; j < V; ++j) z[j] = 0.0f;
      gv[i] = IO::pack(z);
      bv[i] = IO::pack(z);
    }
  }

  for (uint64_t row0 = static_cast<uint64_t>(blockIdx.x) * GROUPS; row0 < rows;
       row0 += static_cast<uint64_t>(gridDim.x) * GROUPS) {
    const uint64_t row = row0 + g;
    const bool live = row < rows;
    const T* xr = x + row * cols;
    T* yr = y + row * cols;

    float v[VPT][V];
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const uint32_t idx = t + i * TPR;
      if (live && idx < nvec) {
        IO::unpack(IO::load(xr, idx), v[i]);
      } else {
#pragma unroll
        for (int j = 0; j < V; ++j) v[i][j] = 0.0f;
      }
    }

    float s = 0.0f;
#pragma unroll
    for (int i = 0; i < VPT; ++i)
#pragma unroll
      for (int j = 0; j < V; ++j) s += v[i][j];
    s = group_allreduce<OpSum, TPR>(s, slots[0], g);
    const float mean = s / n;

    float q = 0.0f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const uint32_t idx = t + i * TPR;
      if (idx < nvec) {  // padded points never reach the lambda (design/tca.md:297-299)
#pragma unroll
        for (int j = 0; j < V; ++j) {
          v[i][j] -= mean;
          q += v[i][j] * v[i][j];
        }
      }
    }
    q = group_allreduce<OpSum, TPR>(q, slots[1], g);
    const float rstd = 1.0f / sqrtf(q / n + eps);

#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const uint32_t idx = t + i * TPR;
      if (live && idx < nvec) {
        float gf[V], bf[V];
        if constexpr (CACHE_GB) {
          IO::unpack(gv[i], gf);
          IO::unpack(bv[i], bf);
        } else {
          IO::unpack(IO::load_keep(gamma, idx), gf);
          IO::unpack(IO::load_keep(beta, idx), bf);
        }
#pragma unroll
        for (int j = 0; j < V; ++j) v[i][j] = v[i][j] * rstd * gf[j] + bf[j];
        IO::store(yr, idx, IO::pack(v[i]));
      }
    }
  }
}

// Rows whose length is not a multiple of a 16-byte vector (E = 4 fp32 or 8 bf16 columns). The flat array's
// vectors still line up, so a row is read as up to E-1 leading elements, the aligned vectors inside it and up
// to E-1 trailing elements (threads 0..2E-3 of the row's group carry one edge element each). gamma and beta
// are aligned to column 0, not to the row's first vector: the E columns under the x vector idx are the
// columns lead + E*idx .., which straddle two of gamma's vectors; both are loaded through L1 and the wanted
// E columns are shifted out of the eight 32-bit words in registers (a 16-bit funnel shift for an odd bf16
// lead, then selects by the two bits of the word shift). Same statistics as layernorm_rows_reg. Without this
// such rows fall to 4- and 2-byte accesses: 2.3-4.4 TB/s fp32 and 1.2-2.5 TB/s bf16 at 1001..50001 columns.
template <typename T>
struct RowEdges {
  static constexpr int E = 16 / sizeof(T);
  const T* xa;    // the first aligned vector inside the row
  T* ya;
  const T* xrow;
  T* yrow;
  uint32_t lead, nint, tail;
  __device__ __forceinline__ RowEdges(const T* x, T* y, uint64_t row, uint32_t cols) {
    const uint64_t first = row * cols;
    lead = static_cast<uint32_t>((E - (first & (E - 1))) & (E - 1));
    if (lead > cols) lead = cols;
    nint = (cols - lead) / E;
    tail = cols - lead - E * nint;
    xrow = x + first;
    yrow = y + first;
    xa = xrow + lead;
    ya = yrow + lead;
  }
  // the column of the edge element thread t of the group carries (0..E-2 lead, E-1..2E-3 tail), or -1
  __device__ __forceinline__ int edge_column(int t) const {
    if (t < E - 1) return t < static_cast<int>(lead) ? t : -1;
    if (t < 2 * (E - 1)) return t - (E - 1) < static_cast<int>(tail) ? static_cast<int>(lead + E * nint) + t - (E - 1) : -1;
    return -1;
  }
};

// The aligned vector k of a parameter row of `cols` elements as four words; columns past the end read as zero.
template <typename T>
__device__ __forceinline__ void param_words(const T* p, uint32_t k, uint32_t cols, uint32_t* w) {
  constexpr int E = 16 / sizeof(T);
  if (static_cast<uint64_t>(k + 1) * E <= cols) {
    const uint4 q = __ldg(reinterpret_cast<const uint4*>(p) + k);
    w[0] = q.x; w[1] = q.y; w[2] = q.z; w[3] = q.w;
  } else {
#pragma unroll
    for (int j = 0; j < 4; ++j) w[j] = 0;
    if constexpr (sizeof(T) == 4) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint64_t c = static_cast<uint64_t>(k) * 4 + j;
        if (c < cols) w[j] = __float_as_uint(__ldg(reinterpret_cast<const float*>(p) + c));
      }
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const uint64_t c = static_cast<uint64_t>(k) * 8 + j;
        if (c < cols) w[j / 2] |= static_cast<uint32_t>(__ldg(reinterpret_cast<const unsigned short*>(p) + c)) << (16 * (j & 1));
      }
    }
  }
}

// E parameter columns starting `lead` columns into the aligned vector idx, as floats.
template <typename T>
__device__ __forceinline__ void param_shifted(const T* p, uint32_t idx, uint32_t lead, uint32_t cols, float* f) {
  uint32_t w[8];
  param_words(p, idx, cols, w);
  param_words(p, idx + 1, cols, w + 4);
  uint32_t words = lead;
  if constexpr (sizeof(T) == 2) {
    const uint32_t half = (lead & 1) * 16;
#pragma unroll
    for (int k = 0; k < 7; ++k) w[k] = __funnelshift_r(w[k], w[k + 1], half);
    words = lead >> 1;
  }
#pragma unroll
  for (int k = 0; k < 5; ++k) w[k] = (words & 2) ? w[k + 2] : w[k];
#pragma unroll
  for (int k = 0; k < 4; ++k) w[k] = (words & 1) ? w[k + 1] : w[k];
  if constexpr (sizeof(T) == 4) {
#pragma unroll
    for (int k = 0; k < 4; ++k) f[k] = __uint_as_float(w[k]);
  } else {
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      f[2 * k] = __uint_as_float(w[k] << 16);
      f[2 * k + 1] = __uint_as_float(w[k] & 0xffff0000u);
    }
  }
}

// Resident threads per SM the unaligned kernel is compiled for: the shift holds sixteen parameter words on top
// of the row, so a thread with 16 fp32 values fits 48 registers, one with 32 values 64, one with 64 values 128.
template <typename T>
constexpr int unaligned_threads_per_sm(int tpr, int vpt) {
  const int values = vpt * static_cast<int>(16 / sizeof(T));
  const int want = values <= 16 ? 1280 : values <= 32 ? 1024 : 512;
  return tpr > want ? tpr : want;
}

template <typename T, int TPR, int VPT>
__global__ void __launch_bounds__(row_cta_threads(TPR), unaligned_threads_per_sm<T>(TPR, VPT) / row_cta_threads(TPR))
layernorm_rows_reg_unaligned(const T* __restrict__ x, const T* __restrict__ gamma, const T* __restrict__ beta,
                             float eps, T* __restrict__ y, uint64_t rows, uint32_t cols) {
  constexpr int THREADS = row_cta_threads(TPR);
  constexpr int GROUPS = THREADS / TPR;
  constexpr int V = 16 / sizeof(T);
  static_assert(TPR >= 2 * (V - 1), "one thread of the group per edge element");
  using IO = VecIO<T, V>;
  using IO1 = VecIO<T, 1>;
  __shared__ float slots[2][32];
  const int g = threadIdx.x / TPR;
  const int t = threadIdx.x % TPR;
  const float n = static_cast<float>(cols);

  for (uint64_t row0 = static_cast<uint64_t>(blockIdx.x) * GROUPS; row0 < rows;
       row0 += static_cast<uint64_t>(gridDim.x) * GROUPS) {
    const uint64_t row = row0 + g;
    const bool live = row < rows;
    const RowEdges<T> r(x, y, live ? row : 0, cols);
    const int ec = live ? r.edge_column(t) : -1;
    float edge = 0.0f;
    if (ec >= 0) IO1::unpack(IO1::load(r.xrow, ec), &edge);

    float v[VPT][V];
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const uint32_t idx = t + i * TPR;
      if (live && idx < r.nint) {
        IO::unpack(IO::load(r.xa, idx), v[i]);
      } else {
#pragma unroll
        for (int j = 0; j < V; ++j) v[i][j] = 0.0f;
      }
    }

    float s = edge;
#pragma unroll
    for (int i = 0; i < VPT; ++i)
#pragma unroll
      for (int j = 0; j < V; ++j) s += v[i][j];
    s = group_allreduce<OpSum, TPR>(s, slots[0], g);
    const float mean = s / n;

    float q = 0.0f;
    if (ec >= 0) {
      edge -= mean;
      q = edge * edge;
    }
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const uint32_t idx = t + i * TPR;
      if (idx < r.nint) {
#pragma unroll
        for (int j = 0; j < V; ++j) {
          v[i][j] -= mean;
          q += v[i][j] * v[i][j];
        }
      }
    }
    q = group_allreduce<OpSum, TPR>(q, slots[1], g);
    const float rstd = 1.0f / sqrtf(q / n + eps);

    if (ec >= 0) {
      float gf, bf;
      IO1::unpack(IO1::load_keep(gamma, ec), &gf);
      IO1::unpack(IO1::load_keep(beta, ec), &bf);
      edge = edge * rstd * gf + bf;
      IO1::store(r.yrow, ec, IO1::pack(&edge));
    }
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const uint32_t idx = t + i * TPR;
      if (live && idx < r.nint) {
        float gf[V], bf[V];
        param_shifted(gamma, idx, r.lead, cols, gf);
        param_shifted(beta, idx, r.lead, cols, bf);
#pragma unroll
        for (int j = 0; j < V; ++j) v[i][j] = v[i][j] * rstd * gf[j] + bf[j];
        IO::store(r.ya, idx, IO::pack(v[i]));
      }
    }
  }
}

template <typename T, int TPR, int VPT>
int launch_reg_unaligned(const T* x, const T* gamma, const T* beta, float eps, T* y, uint64_t rows, uint32_t cols,
                         cudaStream_t s) {
  constexpr int THREADS = row_cta_threads(TPR);
  constexpr int GROUPS = THREADS / TPR;
  uint64_t grid = (rows + GROUPS - 1) / GROUPS;
  if (grid > 0x7fffffffull) grid = 0x7fffffffull;
  layernorm_rows_reg_unaligned<T, TPR, VPT><<<static_cast<unsigned>(grid), THREADS, 0, s>>>(x, gamma, beta, eps, y, rows, cols);
  count_launch();
  return check_launch("layernorm_rows_reg_unaligned");
}

// A row too long for one CTA's registers, cut over a thread-block cluster (see softmax_rows.cu): every
// CTA keeps its segment in registers; the partial sums meet through distributed shared memory.
template <typename T, int THREADS, int VPT, int V>
__global__ void __launch_bounds__(THREADS)
layernorm_rows_cluster(const T* __restrict__ x, const T* __restrict__ gamma, const T* __restrict__ beta, float eps,
                       T* __restrict__ y, uint32_t cols, uint32_t cs, uint32_t seg_vecs) {
  using IO = VecIO<T, V>;
  __shared__ float slots[2][32];
  __shared__ float cl_sum, cl_sq;
  const uint32_t rank = cluster_rank();
  const uint64_t row = blockIdx.x / cs;
  const uint32_t nvec = cols / V;
  const uint32_t v0 = rank * seg_vecs;
  const uint32_t v1 = (nvec - (v0 < nvec ? v0 : nvec) < seg_vecs) ? nvec : v0 + seg_vecs;
  const float n = static_cast<float>(cols);
  const T* xr = x + row * cols;
  T* yr = y + row * cols;

  float v[VPT][V];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const uint32_t idx = v0 + threadIdx.x + i * THREADS;
    if (idx < v1) {
      IO::unpack(IO::load(xr, idx), v[i]);
    } else {
#pragma unroll
      for (int j = 0; j < V; ++j) v[i][j] = 0.0f;
    }
  }
  float s = 0.0f;
#pragma unroll
  for (int i = 0; i < VPT; ++i)
#pragma unroll
    for (int j = 0; j < V; ++j) s += v[i][j];
  s = cta_allreduce<OpSum, THREADS / 32>(s, slots[0]);
  if (threadIdx.x == 0) cl_sum = s;
  cluster_sync_all();
  float gs = 0.0f;
  for (uint32_t r = 0; r < cs; ++r) gs += ld_dsmem(&cl_sum, r);
  const float mean = gs / n;

  float q = 0.0f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const uint32_t idx = v0 + threadIdx.x + i * THREADS;
    if (idx < v1) {
#pragma unroll
      for (int j = 0; j < V; ++j) {
        v[i][j] -= mean;
        q += v[i][j] * v[i][j];
      }
    }
  }
  q = cta_allreduce<OpSum, THREADS / 32>(q, slots[1]);
  if (threadIdx.x == 0) cl_sq = q;
  cluster_sync_all();
  float gq = 0.0f;
  for (uint32_t r = 0; r < cs; ++r) gq += ld_dsmem(&cl_sq, r);
  const float rstd = 1.0f / sqrtf(gq / n + eps);

#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const uint32_t idx = v0 + threadIdx.x + i * THREADS;
    if (idx < v1) {
      float gf[V], bf[V];
      IO::unpack(IO::load_keep(gamma, idx), gf);
      IO::unpack(IO::load_keep(beta, idx), bf);
#pragma unroll
      for (int j = 0; j < V; ++j) v[i][j] = v[i][j] * rstd * gf[j] + bf[j];
      IO::store(yr, idx, IO::pack(v[i]));
    }
  }
  cluster_sync_all();  // no CTA leaves while a peer may still read its partials
}

template <typename T, int THREADS, int VPT, int V>
int launch_cluster_shape(const T* x, const T* gamma, const T* beta, float eps, T* y, uint64_t rows, uint32_t cols,
                         uint32_t nvec, cudaStream_t s) {
  constexpr uint32_t kPerCta = THREADS * VPT;
  // the smallest cluster (2..8 CTAs, any size) whose CTAs cover the row
  uint32_t cs = (nvec + kPerCta - 1) / kPerCta;
  if (cs < 2) cs = 2;
  if (cs > 8) cs = 8;
  const uint32_t seg = (nvec + cs - 1) / cs;
  auto* fn = layernorm_rows_cluster<T, THREADS, VPT, V>;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(rows * cs));
  cfg.blockDim = dim3(THREADS);
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cs;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, fn, x, gamma, beta, eps, y, cols, cs, seg);
  count_launch();
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(TCAB_ERR_CUDA, "layernorm_rows_cluster: launch failed: %s", cudaGetErrorString(e));
  }
  return TCAB_OK;
}

template <typename T, int V>
int launch_cluster(const T* x, const T* gamma, const T* beta, float eps, T* y, uint64_t rows, uint32_t cols,
                   uint32_t nvec, cudaStream_t s) {
  const Tune& tn = tune(kLayernorm);
  // 512 threads x 8 vectors per CTA; the 256-thread shapes (tune p2 = 4 / 8 vectors per thread, for sweeps)
  // measured slower for layer-norm
  if (tn.p2 == 4 && nvec <= 8u * 256u * 4u) return launch_cluster_shape<T, 256, 4, V>(x, gamma, beta, eps, y, rows, cols, nvec, s);
  if (tn.p2 == 8 && nvec <= 8u * 256u * 8u) return launch_cluster_shape<T, 256, 8, V>(x, gamma, beta, eps, y, rows, cols, nvec, s);
  return launch_cluster_shape<T, 512, 8, V>(x, gamma, beta, eps, y, rows, cols, nvec, s);
}

// Long rows streamed by a cluster (the scheme of softmax_rows_cluster_stream): one segment per CTA, nothing kept
// on chip. Pass 1 takes the sums of d = x - K and of d * d with K the row's first element; the CTAs' pairs meet
// through distributed shared memory: mean = K + S1 / n, variance = S2 / n - (S1 / n)^2. When K turns out further
// than one standard deviation from the mean that difference has cancelled digits, and one more pass over the
// (L2-resident) segment takes the centred squares instead. The last pass reads the segment again from L2,
// normalises, scales, shifts and stores. HBM sees each element once in and once out.
template <typename T, int THREADS, int U, int V>
__global__ void __launch_bounds__(THREADS)
layernorm_rows_cluster_stream(const T* __restrict__ x, const T* __restrict__ gamma, const T* __restrict__ beta,
                              float eps, T* __restrict__ y, uint32_t cols, uint32_t cs, uint32_t seg_vecs) {
  using IO = VecIO<T, V>;
  __shared__ float slots[2][32];
  __shared__ float cl_a[2], cl_b;  // this CTA's partials, read by the whole cluster
  const uint32_t rank = cluster_rank();
  const uint64_t row = blockIdx.x / cs;
  const uint32_t nvec = cols / V;
  const uint32_t v0 = rank * seg_vecs < nvec ? rank * seg_vecs : nvec;
  const uint32_t v1 = nvec - v0 < seg_vecs ? nvec : v0 + seg_vecs;
  const float n = static_cast<float>(cols);
  const T* xr = x + row * cols;
  T* yr = y + row * cols;
  float k0[V];
  IO::unpack(IO::load_keep(xr, 0), k0);
  const float K = k0[0];

  float s1 = 0.0f, s2 = 0.0f;
  for (uint32_t base = v0 + threadIdx.x; base < v1; base += THREADS * U) {
    float f[U][V];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint32_t idx = base + u * THREADS;
      if (idx < v1) {
        IO::unpack(IO::load_keep(xr, idx), f[u]);
      } else {
#pragma unroll
        for (int j = 0; j < V; ++j) f[u][j] = K;
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u)
#pragma unroll
      for (int j = 0; j < V; ++j) {
        const float d = f[u][j] - K;
        s1 += d;
        s2 += d * d;
      }
  }
  s1 = cta_allreduce<OpSum, THREADS / 32>(s1, slots[0]);
  s2 = cta_allreduce<OpSum, THREADS / 32>(s2, slots[1]);
  if (threadIdx.x == 0) {
    cl_a[0] = s1;
    cl_a[1] = s2;
  }
  cluster_sync_all();
  float g1 = 0.0f, g2 = 0.0f;
  for (uint32_t r = 0; r < cs; ++r) {  // ascending rank: the same totals in every CTA
    g1 += ld_dsmem(&cl_a[0], r);
    g2 += ld_dsmem(&cl_a[1], r);
  }
  const float delta = g1 / n;
  const float mean = K + delta;
  float var = g2 / n - delta * delta;
  if (!(delta * delta <= var)) {  // K is far from the mean (or something is not finite): centred squares, one more pass
    float q = 0.0f;
    for (uint32_t base = v0 + threadIdx.x; base < v1; base += THREADS * U) {
      float f[U][V];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const uint32_t idx = base + u * THREADS;
        if (idx < v1) {
          IO::unpack(IO::load_keep(xr, idx), f[u]);
        } else {
#pragma unroll
          for (int j = 0; j < V; ++j) f[u][j] = mean;
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u)
#pragma unroll
        for (int j = 0; j < V; ++j) q += (f[u][j] - mean) * (f[u][j] - mean);
    }
    q = cta_allreduce<OpSum, THREADS / 32>(q, slots[0]);  // every thread has read slots[0] before the cluster barrier above
    if (threadIdx.x == 0) cl_b = q;
    cluster_sync_all();
    float gq = 0.0f;
    for (uint32_t r = 0; r < cs; ++r) gq += ld_dsmem(&cl_b, r);
    var = gq / n;
  }
  const float rstd = 1.0f / sqrtf(var + eps);
  for (uint32_t base = v0 + threadIdx.x; base < v1; base += THREADS * U) {
    float f[U][V];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint32_t idx = base + u * THREADS;
      if (idx < v1) IO::unpack(IO::load(xr, idx), f[u]);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint32_t idx = base + u * THREADS;
      if (idx < v1) {
        float gf[V], bf[V];
        IO::unpack(IO::load_keep(gamma, idx), gf);
        IO::unpack(IO::load_keep(beta, idx), bf);
#pragma unroll
        for (int j = 0; j < V; ++j) f[u][j] = (f[u][j] - mean) * rstd * gf[j] + bf[j];
        IO::store(yr, idx, IO::pack(f[u]));
      }
    }
  }
  cluster_sync_all();  // no CTA leaves while a peer may still read its partials
}

template <typename T, int THREADS, int U, int V>
int launch_cluster_stream_shape(const T* x, const T* gamma, const T* beta, float eps, T* y, uint64_t rows, uint32_t cols,
                                uint32_t nvec, uint32_t cs, cudaStream_t s) {
  const uint32_t seg = (nvec + cs - 1) / cs;
  auto* fn = layernorm_rows_cluster_stream<T, THREADS, U, V>;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(rows * cs));
  cfg.blockDim = dim3(THREADS);
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cs;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, fn, x, gamma, beta, eps, y, cols, cs, seg);
  count_launch();
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(TCAB_ERR_CUDA, "layernorm_rows_cluster_stream: launch failed: %s", cudaGetErrorString(e));
  }
  return TCAB_OK;
}

// tune("layernorm", _, p1 = CTAs per row, p2 = shape 1..5, p3 = 7) forces a shape of the streaming clusters.
template <typename T, int V>
int launch_cluster_stream(const T* x, const T* gamma, const T* beta, float eps, T* y, uint64_t rows, uint32_t cols,
                          uint32_t nvec, bool few_rows, cudaStream_t s) {
  const Tune& tn = tune(kLayernorm);
  uint32_t cs = 0;
  int shape = 0;
  if (tn.p3 == 7) {
    cs = tn.p1 >= 1 && tn.p1 <= 8 ? static_cast<uint32_t>(tn.p1) : 0u;
    shape = tn.p2;
  }
  if (shape <= 0 && few_rows) {
    shape = 2;
    if (cs == 0) cs = 8;
  }
  if (shape <= 0) shape = nvec <= 8u * 1024u * 4u ? 1 : nvec <= 8u * 2048u * 4u ? 2 : 5;
  if (cs == 0) cs = stream_cluster_size(nvec, shape == 1 ? 1024u : shape == 5 ? 4096u : 2048u, sizeof(T) == 4);
  switch (shape) {
    case 1: return launch_cluster_stream_shape<T, 256, 4, V>(x, gamma, beta, eps, y, rows, cols, nvec, cs, s);
    case 2: return launch_cluster_stream_shape<T, 512, 4, V>(x, gamma, beta, eps, y, rows, cols, nvec, cs, s);
    case 3: return launch_cluster_stream_shape<T, 256, 8, V>(x, gamma, beta, eps, y, rows, cols, nvec, cs, s);
    case 4: return launch_cluster_stream_shape<T, 256, 2, V>(x, gamma, beta, eps, y, rows, cols, nvec, cs, s);
    default: return launch_cluster_stream_shape<T, 512, 8, V>(x, gamma, beta, eps, y, rows, cols, nvec, cs, s);
  }
}

// Rows too long even for a cluster: one CTA per row, three streaming passes (sum,
// centred squares, normalise); passes two and three re-read the row from L2.
template <typename T, int THREADS, int V>
__global__ void __launch_bounds__(THREADS)
layernorm_rows_stream(const T* __restrict__ x, const T* __restrict__ gamma, const T* __restrict__ beta,
                      float eps, T* __restrict__ y, uint64_t rows, uint32_t cols) {
  using IO = VecIO<T, V>;
  __shared__ float slots[2][32];
  const uint32_t nvec = cols / V;
  const float n = static_cast<float>(cols);
  for (uint64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* xr = x + row * cols;
    T* yr = y + row * cols;
    float s = 0.0f;
    for (uint32_t idx = threadIdx.x; idx < nvec; idx += THREADS) {
      float f[V];
      IO::unpack(IO::load_keep(xr, idx), f);
#pragma unroll
      for (int j = 0; j < V; ++j) s += f[j];
    }
    const float mean = cta_allreduce<OpSum, THREADS / 32>(s, slots[0]) / n;
    float q = 0.0f;
    for (uint32_t idx = threadIdx.x; idx < nvec; idx += THREADS) {
      float f[V];
      IO::unpack(IO::load_keep(xr, idx), f);
#pragma unroll
      for (int j = 0; j < V; ++j) q += (f[j] - mean) * (f[j] - mean);
    }
    const float rstd = 1.0f / sqrtf(cta_allreduce<OpSum, THREADS / 32>(q, slots[1]) / n + eps);
    for (uint32_t idx = threadIdx.x; idx < nvec; idx += THREADS) {
      float f[V], gf[V], bf[V];
      IO::unpack(IO::load(xr, idx), f);
      IO::unpack(IO::load_keep(gamma, idx), gf);
      IO::unpack(IO::load_keep(beta, idx), bf);
#pragma unroll
      for (int j = 0; j < V; ++j) f[j] = (f[j] - mean) * rstd * gf[j] + bf[j];
      IO::store(yr, idx, IO::pack(f));
    }
    __syncthreads();
  }
}

template <typename T, int TPR, int VPT, int V, bool CACHE_GB>
int launch_reg2(const T* x, const T* gamma, const T* beta, float eps, T* y, uint64_t rows, uint32_t cols,
                int ctas_per_sm, cudaStream_t s) {
  constexpr int THREADS = row_cta_threads(TPR);
  constexpr int GROUPS = THREADS / TPR;
  auto* fn = layernorm_rows_reg<T, TPR, VPT, V, CACHE_GB>;
  // One CTA per group of rows (see softmax_rows.cu: the hardware block scheduler staggers the CTAs,
  // a persistent grid runs them in lock step); a positive ctas_per_sm caps the grid.
  const uint64_t need = (rows + GROUPS - 1) / GROUPS;
  uint64_t grid = ctas_per_sm > 0 ? static_cast<uint64_t>(sm_count()) * ctas_per_sm : need;
  if (grid > need) grid = need;
  if (grid > 0x7fffffffull) grid = 0x7fffffffull;
  fn<<<static_cast<unsigned>(grid), THREADS, 0, s>>>(x, gamma, beta, eps, y, rows, cols);
  count_launch();
  return check_launch("layernorm_rows_reg");
}

// tune p3 == 1 selects the register-cached gamma/beta variant.
template <typename T, int TPR, int VPT, int V>
int launch_reg(const T* x, const T* gamma, const T* beta, float eps, T* y, uint64_t rows, uint32_t cols,
               int ctas_per_sm, cudaStream_t s) {
  if (tune(kLayernorm).p3 == 1)
    return launch_reg2<T, TPR, VPT, V, true>(x, gamma, beta, eps, y, rows, cols, ctas_per_sm, s);
  return launch_reg2<T, TPR, VPT, V, false>(x, gamma, beta, eps, y, rows, cols, ctas_per_sm, s);
}

#define TCAB_LN_SHAPES_BASE(X) \
  X(1, 1) X(2, 1) X(4, 1) X(8, 1) X(8, 2) X(8, 4) X(16, 4) X(32, 4) X(64, 4) X(128, 4) X(256, 4) X(512, 4) X(1024, 4) \
  X(1024, 8) X(1024, 16)
#define TCAB_LN_SHAPES_EXTRA(X) \
  X(32, 32) X(64, 16) X(128, 8) X(512, 2) X(1024, 1) X(256, 8) X(512, 8) X(64, 8) X(128, 2) X(256, 2) \
  X(16, 5) X(32, 5) X(64, 5) X(128, 5) X(256, 5) X(16, 3) X(32, 3) X(64, 3) X(128, 3) X(256, 3) X(512, 3)

inline int launch_smem(const __nv_bfloat16* x, const __nv_bfloat16* gamma, const __nv_bfloat16* beta, float eps,
                       __nv_bfloat16* y, uint64_t rows, uint32_t cols, cudaStream_t s) {
  return launch_layernorm_rows_smem_bf16(x, gamma, beta, eps, y, rows, cols, s);
}
inline int launch_smem(const float* x, const float* gamma, const float* beta, float eps, float* y, uint64_t rows,
                       uint32_t cols, cudaStream_t s) {
  return launch_layernorm_rows_smem_f32(x, gamma, beta, eps, y, rows, cols, s);
}

template <typename T, int VW>
int dispatch(const T* x, const T* gamma, const T* beta, float eps, T* y, uint64_t rows, uint32_t cols,
             cudaStream_t s) {
  if (rows == 0 || cols == 0) return TCAB_OK;
  const bool vec = (cols % VW == 0) && aligned16(x) && aligned16(y) && aligned16(gamma) && aligned16(beta);
  const uint32_t nvec = vec ? cols / VW : cols;
  const Tune& tn = tune(kLayernorm);
  // rows that are not whole 16-byte vectors but still fit a CTA's registers as such (p3 == 6: 4- / 2-byte path)
  if (cols % VW != 0 && cols >= 4u * VW && aligned16(x) && aligned16(y) && aligned16(gamma) && aligned16(beta) &&
      tn.p0 <= 0 && tn.p3 != 6) {
    int ut = 0, uv = 0;
    if (choose_row_shape_fit(cols / VW, true, true, VW, &ut, &uv) && ut >= 2 * (VW - 1)) {
#define TCAB_CASE(TP, P) \
  if constexpr (TP >= 2 * (VW - 1) && (TP < 1024 || P * VW <= 32)) /* longer rows would spill */ \
    if (ut == TP && uv == P) return launch_reg_unaligned<T, TP, P>(x, gamma, beta, eps, y, rows, cols, s);
      TCAB_CASE(8, 1) TCAB_CASE(8, 2) TCAB_CASE(8, 4) TCAB_CASE(16, 4) TCAB_CASE(32, 4) TCAB_CASE(64, 4) TCAB_CASE(128, 4)
      TCAB_CASE(256, 4) TCAB_CASE(512, 4) TCAB_CASE(1024, 4) TCAB_CASE(128, 8) TCAB_CASE(256, 8) TCAB_CASE(512, 8)
      TCAB_CASE(64, 8) TCAB_CASE(1024, 8) TCAB_CASE(1024, 16)
#undef TCAB_CASE
    }
  }
  int tpr = 0, vpt = 0;
  bool fits = layernorm_row_shape(nvec, vec, static_cast<int>(sizeof(T)), &tpr, &vpt);
  if (tn.p0 > 0 && tn.p1 > 0 && static_cast<uint64_t>(tn.p0) * tn.p1 >= nvec) {
    tpr = tn.p0;
    vpt = tn.p1;
    fits = true;
  }
  // Long rows with enough of them to fill the GPU: the shared-memory kernel (rows_smem.cu). fp32 from 2560
  // vectors on (10240 columns: 5.7 TB/s with three CTAs per SM, 3.8 for the 1024-thread register kernel; 4.9-5.0
  // up to 45056 columns). For bf16, unpacking is the cost of a pass: its kernel takes mean and variance from one
  // pass (shifted sums) and wins where the register kernel needs 1024 threads, rows beyond 32 KiB (20480 columns
  // 4.9 against 3.8, 24576 columns 5.0 against 4.0, 32768 columns 4.5 against 4.2, 65536 columns 4.0 against 3.9,
  // 90112 columns 3.9 against 2.0). p3 == 4 forces the shared-memory kernel.
  // Long rows, enough of them to fill the GPU with small CTAs: streaming clusters. fp32 from 24576 columns
  // (measured, 2^27 elements, TB/s against the shared-memory rows / register kernels: 24576 columns 5.5 against
  // 4.9, 32768 5.2 against 5.0, 45056 5.3 against 4.6, 65536 4.9 against 3.7, 131072 4.9 against 3.0); bf16 rows
  // only beyond what the shared-memory kernel takes (131072 columns 4.2 against 2.4; at 49152-65536 the two are
  // within 5 %). p3 == 7 forces them.
  {
    const uint64_t rb = static_cast<uint64_t>(cols) * sizeof(T);
    const bool pays = sizeof(T) == 4 ? nvec >= 6144u : !rows_smem_fits(rb);
    // Fewer rows: beyond what the register clusters take (16384 vectors) eight CTAs of 512 threads stream a row
    // (fp32 64 x 262144: 3.3 against 1.4 TB/s for the one-CTA kernel, 16 x 1048576: 2.2 against 0.4).
    const bool many = rows * 2 >= static_cast<uint64_t>(sm_count());
    const bool few_long = !many && nvec > 16384u;
    if (vec && tn.p0 <= 0 && rows * 8 <= 0x7fffffffull &&
        (tn.p3 == 7 || (tn.p3 <= 0 && ((pays && many) || few_long))))
      return launch_cluster_stream<T, VW>(x, gamma, beta, eps, y, rows, cols, nvec, few_long, s);
  }
  const uint64_t row_bytes = static_cast<uint64_t>(cols) * sizeof(T);
  const bool smem_pays = sizeof(T) == 4 ? nvec >= 2560 : row_bytes > 32768;
  if (vec && tn.p0 <= 0 && rows_smem_fits(row_bytes) &&
      (tn.p3 == 4 || (tn.p3 <= 0 && smem_pays && rows >= static_cast<uint64_t>(sm_count()))))
    return launch_smem(x, gamma, beta, eps, y, rows, cols, s);
  // Few long rows go to the cluster kernel (2-8 CTAs x 4096 vectors share a row, so a handful of rows
  // still spreads over the GPU: 64 x 131072 bf16 runs at 1.75 TB/s instead of 1.10). With many rows the
  // single-CTA kernels are faster (4.3 vs 2.6 TB/s at 4096 x 65536: three cluster barriers per row are
  // not hidden), so the cluster is used only while the rows alone cannot fill the SMs. p3 == 3 forces it.
  const bool few_rows = rows < 2ull * sm_count() && nvec > 8192;
  if (tn.p0 <= 0 && nvec > (tn.p3 == 3 ? 1024u : 4096u) && nvec <= 8u * 4096u && rows * 8 <= 0x7fffffffull && tn.p3 != 2 &&
      ((few_rows && nvec <= 16384) || tn.p3 == 3))
    return vec ? launch_cluster<T, VW>(x, gamma, beta, eps, y, rows, cols, nvec, s)
               : launch_cluster<T, 1>(x, gamma, beta, eps, y, rows, cols, nvec, s);
  if (fits) {
#define TCAB_CASE(TP, P)                                                                         \
  if (tpr == TP && vpt == P)                                                                     \
    return vec ? launch_reg<T, TP, P, VW>(x, gamma, beta, eps, y, rows, cols, tn.p2, s)          \
               : launch_reg<T, TP, P, 1>(x, gamma, beta, eps, y, rows, cols, tn.p2, s);
    TCAB_LN_SHAPES_BASE(TCAB_CASE)
#undef TCAB_CASE
#define TCAB_CASE(TP, P) \
  if (vec && tpr == TP && vpt == P) return launch_reg<T, TP, P, VW>(x, gamma, beta, eps, y, rows, cols, tn.p2, s);
    TCAB_LN_SHAPES_EXTRA(TCAB_CASE)
#undef TCAB_CASE
    if (tn.p0 > 0) return fail(TCAB_ERR_UNSUPPORTED, "layernorm: no kernel for tuned shape %d x %d", tpr, vpt);
  }
  constexpr int THREADS = 512;
  const uint64_t cap = static_cast<uint64_t>(sm_count()) * 4;
  const unsigned grid = static_cast<unsigned>(rows < cap ? rows : cap);
  if (vec) {
    layernorm_rows_stream<T, THREADS, VW><<<grid, THREADS, 0, s>>>(x, gamma, beta, eps, y, rows, cols);
  } else {
    layernorm_rows_stream<T, THREADS, 1><<<grid, THREADS, 0, s>>>(x, gamma, beta, eps, y, rows, cols);
  }
  count_launch();
  return check_launch("layernorm_rows_stream");
}

}  // namespace

int launch_layernorm_rows_bf16(const __nv_bfloat16* x, const __nv_bfloat16* gamma,
                               const __nv_bfloat16* beta, float eps, __nv_bfloat16* y,
                               uint64_t rows, uint32_t cols, cudaStream_t s) {
  return dispatch<__nv_bfloat16, 8>(x, gamma, beta, eps, y, rows, cols, s);
}

int launch_layernorm_rows_f32(const float* x, const float* gamma, const float* beta, float eps,
                              float* y, uint64_t rows, uint32_t cols, cudaStream_t s) {
  return dispatch<float, 4>(x, gamma, beta, eps, y, rows, cols, s);
}

}  // namespace tcab
