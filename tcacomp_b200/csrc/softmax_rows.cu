// softmax_rows.cu -- row softmax as ONE fused map | reduce | map kernel.
//
//   m_i = max_j x[i,j];  s_i = sum_j expf(x[i,j] - m_i);  y[i,j] = expf(x[i,j] - m_i) / s_i
//
// The reference cannot store a rank-preserving map (pkg/chain.go:433-438) and
// ships only the reduction core of this chain (testing/kernels/fusion/softmax.tca,
// runner testing/runners/softmax.cu:49-61); its reducers run one shuffle tree and
// two barriers PER ELEMENT (runtime/tca/reducer.h:109-167).
//
// Three kernels:
//   softmax_rows_reg     the row lives in registers (4 vectors of 4 fp32 per thread): x is read from HBM once and
//                        y written once (8 bytes per element, the roofline figure);
//                        one shuffle/shared-memory tree per reduction per ROW.
//   softmax_rows_cluster rows of 32K..256K elements: the row is cut over a thread-block cluster of
//                        2-8 CTAs, each keeps its segment in registers, the partial max and sum
//                        meet through distributed shared memory: still one read and one write.
//   softmax_rows_online  rows too long even for that: a single streaming pass
//                        keeps a running (max, sum) pair per thread, rescaling
//                        the sum when the max moves, then a second pass over the
//                        row (L2-resident for any realistic row) writes y.
// expf is the accurate CUDA expf (no fast-math); y multiplies by 1/s_i, which
// differs from the division by at most 1 ulp.
#include "rowvec.cuh"

namespace tcab {
namespace {

template <int TPR, int VPT, int V>
__global__ void __launch_bounds__(row_cta_threads(TPR), row_min_ctas(TPR, VPT * V, 16, 1536))
softmax_rows_reg(const float* __restrict__ x, float* __restrict__ y, uint64_t rows, uint32_t cols) {
  constexpr int THREADS = row_cta_threads(TPR);
  constexpr int GROUPS = THREADS / TPR;
  using IO = VecIO<float, V>;
  __shared__ float slots[2][32];

  const int g = threadIdx.x / TPR;
  const int t = threadIdx.x % TPR;
  const uint32_t nvec = cols / V;
  const int used = static_cast<int>((nvec + TPR - 1) / TPR);

  for (uint64_t row0 = static_cast<uint64_t>(blockIdx.x) * GROUPS; row0 < rows;
       row0 += static_cast<uint64_t>(gridDim.x) * GROUPS) {
    const uint64_t row = row0 + g;
    const bool live = row < rows;
    const float* xr = x + row * cols;
    float* yr = y + row * cols;

    // `used` vector slots of each thread can hold data for this row length (the same for every thread);
    // the slots beyond it are skipped as a whole, so a row shorter than TPR * VPT vectors costs no
    // arithmetic for the padding
    float v[VPT][V];
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      if (i < used) {
        const uint32_t idx = t + i * TPR;
        if (live && idx < nvec) {
          IO::unpack(IO::load(xr, idx), v[i]);
        } else {
#pragma unroll
          for (int j = 0; j < V; ++j) v[i][j] = -INFINITY;  // identity of max; expf(-inf - m) = 0
        }
      }
    }

    float m = -INFINITY;
#pragma unroll
    for (int i = 0; i < VPT; ++i)
      if (i < used) {
#pragma unroll
        for (int j = 0; j < V; ++j) m = fmaxf(m, v[i][j]);
      }
    m = group_allreduce<OpMax, TPR>(m, slots[0], g);

    float s = 0.0f;
#pragma unroll
    for (int i = 0; i < VPT; ++i)
      if (i < used) {
#pragma unroll
        for (int j = 0; j < V; ++j) {
          v[i][j] = expf(v[i][j] - m);
          s += v[i][j];
        }
      }
    s = group_allreduce<OpSum, TPR>(s, slots[1], g);
    const float inv = 1.0f / s;

#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const uint32_t idx = t + i * TPR;
      if (i < used && live && idx < nvec) {
#pragma unroll
        for (int j = 0; j < V; ++j) v[i][j] *= inv;
        IO::store(yr, idx, IO::pack(v[i]));
      }
    }
  }
}

// Rows whose length is not a multiple of four columns: a row then starts at any 4-byte offset, but the
// 16-byte vectors of the flat array still line up (the base pointer is 16-byte aligned). A row is read as
// up to three leading elements, the aligned vectors inside it (at most cols / 4, so the launch shape is the
// one of an aligned row of that length) and up to three trailing elements; the six edge elements ride in one
// extra value of threads 0..5 of the row's group. Same arithmetic and fold as softmax_rows_reg<TPR, VPT, 4>;
// without this such rows fall to 4-byte loads (2.9 TB/s at 50257 columns).
struct UnalignedRow {
  const float* xa;   // the first aligned vector inside the row
  float* ya;
  const float* xrow; // the row itself
  float* yrow;
  uint32_t lead, nint, tail;
  __device__ __forceinline__ UnalignedRow(const float* x, float* y, uint64_t row, uint32_t cols) {
    const uint64_t first = row * cols;
    lead = static_cast<uint32_t>((4 - (first & 3)) & 3);
    if (lead > cols) lead = cols;
    nint = (cols - lead) / 4;
    tail = cols - lead - 4 * nint;
    xrow = x + first;
    yrow = y + first;
    xa = xrow + lead;
    ya = yrow + lead;
  }
  // the edge element of thread t of the row's group (threads 0..2 lead, 3..5 tail), or -1
  __device__ __forceinline__ int edge_index(int t) const {
    if (t < 3) return t < static_cast<int>(lead) ? t : -1;
    if (t < 6) return t - 3 < static_cast<int>(tail) ? static_cast<int>(lead + 4 * nint) + t - 3 : -1;
    return -1;
  }
};

template <int TPR, int VPT>
__global__ void __launch_bounds__(row_cta_threads(TPR), row_min_ctas(TPR, VPT * 4, 16, 1536))
softmax_rows_reg_unaligned(const float* __restrict__ x, float* __restrict__ y, uint64_t rows, uint32_t cols) {
  constexpr int THREADS = row_cta_threads(TPR);
  constexpr int GROUPS = THREADS / TPR;
  static_assert(TPR >= 8, "six threads of a group carry the edge elements");
  __shared__ float slots[2][32];
  const int g = threadIdx.x / TPR;
  const int t = threadIdx.x % TPR;
  const int used = static_cast<int>((cols / 4 + TPR - 1) / TPR);

  for (uint64_t row0 = static_cast<uint64_t>(blockIdx.x) * GROUPS; row0 < rows;
       row0 += static_cast<uint64_t>(gridDim.x) * GROUPS) {
    const uint64_t row = row0 + g;
    const bool live = row < rows;
    const UnalignedRow r(x, y, live ? row : 0, cols);
    const int ei = live ? r.edge_index(t) : -1;
    float edge = ei >= 0 ? ld_stream(r.xrow + ei) : -INFINITY;

    float v[VPT][4];
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      if (i < used) {
        const uint32_t idx = t + i * TPR;
        if (live && idx < r.nint) {
          const float4 q = ld_stream(reinterpret_cast<const float4*>(r.xa) + idx);
          v[i][0] = q.x; v[i][1] = q.y; v[i][2] = q.z; v[i][3] = q.w;
        } else {
#pragma unroll
          for (int j = 0; j < 4; ++j) v[i][j] = -INFINITY;
        }
      }
    }
    float m = edge;
#pragma unroll
    for (int i = 0; i < VPT; ++i)
      if (i < used) {
#pragma unroll
        for (int j = 0; j < 4; ++j) m = fmaxf(m, v[i][j]);
      }
    m = group_allreduce<OpMax, TPR>(m, slots[0], g);
    edge = expf(edge - m);
    float s = edge;
#pragma unroll
    for (int i = 0; i < VPT; ++i)
      if (i < used) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          v[i][j] = expf(v[i][j] - m);
          s += v[i][j];
        }
      }
    s = group_allreduce<OpSum, TPR>(s, slots[1], g);
    const float inv = 1.0f / s;
    if (ei >= 0) st_stream(r.yrow + ei, edge * inv);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const uint32_t idx = t + i * TPR;
      if (i < used && live && idx < r.nint)
        st_stream(reinterpret_cast<float4*>(r.ya) + idx, make_float4(v[i][0] * inv, v[i][1] * inv, v[i][2] * inv, v[i][3] * inv));
    }
  }
}

template <int TPR, int VPT>
int launch_reg_unaligned(const float* x, float* y, uint64_t rows, uint32_t cols, cudaStream_t s) {
  constexpr int THREADS = row_cta_threads(TPR);
  constexpr int GROUPS = THREADS / TPR;
  uint64_t grid = (rows + GROUPS - 1) / GROUPS;
  if (grid > 0x7fffffffull) grid = 0x7fffffffull;
  softmax_rows_reg_unaligned<TPR, VPT><<<static_cast<unsigned>(grid), THREADS, 0, s>>>(x, y, rows, cols);
  count_launch();
  return check_launch("softmax_rows_reg_unaligned");
}

// A row too long for one CTA's registers is cut over a thread-block CLUSTER of CS CTAs: each CTA
// keeps its segment in registers, the per-CTA max and sum meet through distributed shared memory
// (every CTA reads the CS partials of its peers), so x is still read from HBM exactly once.
template <int CS_MAX, int THREADS, int VPT, int V>
__global__ void __launch_bounds__(THREADS)
softmax_rows_cluster(const float* __restrict__ x, float* __restrict__ y, uint64_t rows, uint32_t cols, uint32_t cs,
                     uint32_t seg_vecs) {
  using IO = VecIO<float, V>;
  __shared__ float slots[2][32];
  __shared__ float cl_max, cl_sum;  // this CTA's partials, read by the whole cluster
  const uint32_t rank = cluster_rank();
  const uint64_t row = blockIdx.x / cs;  // clusters are consecutive CTAs: one row per cluster
  const uint32_t nvec = cols / V;
  const uint32_t v0 = rank * seg_vecs;
  const uint32_t v1 = (nvec - (v0 < nvec ? v0 : nvec) < seg_vecs) ? nvec : v0 + seg_vecs;
  const float* xr = x + row * cols;
  float* yr = y + row * cols;
  (void)rows;

  const int used = static_cast<int>((seg_vecs + THREADS - 1) / THREADS);  // vector slots that can hold data
  float v[VPT][V];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    if (i < used) {
      const uint32_t idx = v0 + threadIdx.x + i * THREADS;
      if (idx < v1) {
        IO::unpack(IO::load(xr, idx), v[i]);
      } else {
#pragma unroll
        for (int j = 0; j < V; ++j) v[i][j] = -INFINITY;
      }
    }
  }
  float m = -INFINITY;
#pragma unroll
  for (int i = 0; i < VPT; ++i)
    if (i < used) {
#pragma unroll
      for (int j = 0; j < V; ++j) m = fmaxf(m, v[i][j]);
    }
  m = cta_allreduce<OpMax, THREADS / 32>(m, slots[0]);
  if (threadIdx.x == 0) cl_max = m;
  cluster_sync_all();
  float gm = -INFINITY;
  for (uint32_t r = 0; r < cs; ++r) gm = fmaxf(gm, ld_dsmem(&cl_max, r));

  float s = 0.0f;
#pragma unroll
  for (int i = 0; i < VPT; ++i)
    if (i < used) {
#pragma unroll
      for (int j = 0; j < V; ++j) {
        v[i][j] = expf(v[i][j] - gm);
        s += v[i][j];
      }
    }
  s = cta_allreduce<OpSum, THREADS / 32>(s, slots[1]);
  if (threadIdx.x == 0) cl_sum = s;
  cluster_sync_all();
  float gs = 0.0f;
  for (uint32_t r = 0; r < cs; ++r) gs += ld_dsmem(&cl_sum, r);  // ascending rank: the same total in every CTA
  const float inv = 1.0f / gs;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const uint32_t idx = v0 + threadIdx.x + i * THREADS;
    if (i < used && idx < v1) {
#pragma unroll
      for (int j = 0; j < V; ++j) v[i][j] *= inv;
      IO::store(yr, idx, IO::pack(v[i]));
    }
  }
  cluster_sync_all();  // no CTA leaves while a peer may still read its partials
}

template <int THREADS, int VPT, int V>
int launch_cluster_shape(const float* x, float* y, uint64_t rows, uint32_t cols, uint32_t nvec, cudaStream_t s) {
  constexpr uint32_t kPerCta = THREADS * VPT;
  // the smallest cluster (2..8 CTAs, any size) whose CTAs cover the row
  uint32_t cs = (nvec + kPerCta - 1) / kPerCta;
  if (cs < 2) cs = 2;
  if (cs > 8) cs = 8;
  const uint32_t seg = (nvec + cs - 1) / cs;
  auto* fn = softmax_rows_cluster<8, THREADS, VPT, V>;
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
  const cudaError_t e = cudaLaunchKernelEx(&cfg, fn, x, y, rows, cols, cs, seg);
  count_launch();
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(TCAB_ERR_CUDA, "softmax_rows_cluster: launch failed: %s", cudaGetErrorString(e));
  }
  return TCAB_OK;
}

// Small CTAs while they cover the row (more of them fit an SM, so a CTA waiting at a cluster barrier
// does not idle the SM); 512 threads x 16 vectors only for the longest rows.
// 8 or 16 vectors per thread for a row of nvec vectors on 256-thread CTAs. Both shapes keep the same bytes in
// registers per SM (four CTAs of 32 KiB or two of 64 KiB), but only while the CTAs are full: the row is cut evenly
// over ceil(nvec / capacity) CTAs, and what a CTA leaves unused is missing from the bytes in flight. Measured
// (2^27 elements, TB/s, 8 against 16 vectors): 24576 columns 5.4 / 5.1, 32768 5.5 / 5.7, 40960 5.2 / 4.8, 49152
// 5.1 / 5.3, 65536 5.0 / 5.3 -- the wider shape wins whenever it fills its CTAs as well as the narrow one, and
// always against clusters of seven or eight narrow CTAs (57344 columns 4.8 / 5.1, 51200 4.4 / 4.8; rounding seven
// CTAs up to eight measured 1-4 % slower, so the size stays the smallest that covers the row). tune("softmax", _, _, p2 = 8 | 16) forces one.
inline bool cluster_wide(uint32_t nvec) {
  const int forced = tune(kSoftmax).p2;
  if (forced == 16) return true;
  if (forced == 8 || nvec <= 4096u) return false;
  const uint32_t cs8 = (nvec + 2047u) / 2048u, cs16 = (nvec + 4095u) / 4096u;
  return cs8 >= 7u || cs8 == 2u * cs16;
}

template <int V>
int launch_cluster(const float* x, float* y, uint64_t rows, uint32_t cols, uint32_t nvec, cudaStream_t s) {
  if (nvec <= 8u * 256u * 8u && !cluster_wide(nvec)) return launch_cluster_shape<256, 8, V>(x, y, rows, cols, nvec, s);
  if (nvec <= 8u * 256u * 16u) return launch_cluster_shape<256, 16, V>(x, y, rows, cols, nvec, s);
  return launch_cluster_shape<512, 16, V>(x, y, rows, cols, nvec, s);
}

// The cluster kernel for rows that are not a multiple of four columns (see softmax_rows_reg_unaligned): the
// aligned vectors inside a row are cut into one segment per CTA; CTA 0 also carries the edge elements.
template <int THREADS, int VPT>
__global__ void __launch_bounds__(THREADS)
softmax_rows_cluster_unaligned(const float* __restrict__ x, float* __restrict__ y, uint32_t cols, uint32_t cs,
                               uint32_t seg_vecs) {
  __shared__ float slots[2][32];
  __shared__ float cl_max, cl_sum;
  const uint32_t rank = cluster_rank();
  const UnalignedRow r(x, y, blockIdx.x / cs, cols);
  const uint32_t v0 = rank * seg_vecs;
  const uint32_t v1 = (r.nint - (v0 < r.nint ? v0 : r.nint) < seg_vecs) ? r.nint : v0 + seg_vecs;
  const int used = static_cast<int>((seg_vecs + THREADS - 1) / THREADS);
  const int ei = rank == 0 ? r.edge_index(static_cast<int>(threadIdx.x)) : -1;
  float edge = ei >= 0 ? ld_stream(r.xrow + ei) : -INFINITY;

  float v[VPT][4];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    if (i < used) {
      const uint32_t idx = v0 + threadIdx.x + i * THREADS;
      if (idx < v1) {
        const float4 q = ld_stream(reinterpret_cast<const float4*>(r.xa) + idx);
        v[i][0] = q.x; v[i][1] = q.y; v[i][2] = q.z; v[i][3] = q.w;
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) v[i][j] = -INFINITY;
      }
    }
  }
  float m = edge;
#pragma unroll
  for (int i = 0; i < VPT; ++i)
    if (i < used) {
#pragma unroll
      for (int j = 0; j < 4; ++j) m = fmaxf(m, v[i][j]);
    }
  m = cta_allreduce<OpMax, THREADS / 32>(m, slots[0]);
  if (threadIdx.x == 0) cl_max = m;
  cluster_sync_all();
  float gm = -INFINITY;
  for (uint32_t k = 0; k < cs; ++k) gm = fmaxf(gm, ld_dsmem(&cl_max, k));
  edge = expf(edge - gm);
  float s = edge;
#pragma unroll
  for (int i = 0; i < VPT; ++i)
    if (i < used) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        v[i][j] = expf(v[i][j] - gm);
        s += v[i][j];
      }
    }
  s = cta_allreduce<OpSum, THREADS / 32>(s, slots[1]);
  if (threadIdx.x == 0) cl_sum = s;
  cluster_sync_all();
  float gs = 0.0f;
  for (uint32_t k = 0; k < cs; ++k) gs += ld_dsmem(&cl_sum, k);
  const float inv = 1.0f / gs;
  if (ei >= 0) st_stream(r.yrow + ei, edge * inv);
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const uint32_t idx = v0 + threadIdx.x + i * THREADS;
    if (i < used && idx < v1)
      st_stream(reinterpret_cast<float4*>(r.ya) + idx, make_float4(v[i][0] * inv, v[i][1] * inv, v[i][2] * inv, v[i][3] * inv));
  }
  cluster_sync_all();  // no CTA leaves while a peer may still read its partials
}

template <int THREADS, int VPT>
int launch_cluster_unaligned(const float* x, float* y, uint64_t rows, uint32_t cols, uint32_t max_nv, cudaStream_t s) {
  constexpr uint32_t kPerCta = THREADS * VPT;
  uint32_t cs = (max_nv + kPerCta - 1) / kPerCta;
  if (cs < 2) cs = 2;
  if (cs > 8) cs = 8;
  const uint32_t seg = (max_nv + cs - 1) / cs;
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
  const cudaError_t e = cudaLaunchKernelEx(&cfg, softmax_rows_cluster_unaligned<THREADS, VPT>, x, y, cols, cs, seg);
  count_launch();
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(TCAB_ERR_CUDA, "softmax_rows_cluster_unaligned: launch failed: %s", cudaGetErrorString(e));
  }
  return TCAB_OK;
}

// One CTA per row, any length. Pass 1 is the single-pass online max/sum.
template <int THREADS, int V>
__global__ void __launch_bounds__(THREADS)
softmax_rows_online(const float* __restrict__ x, float* __restrict__ y, uint64_t rows, uint32_t cols) {
  using IO = VecIO<float, V>;
  __shared__ float slots[2][32];
  const uint32_t nvec = cols / V;
  for (uint64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const float* xr = x + row * cols;
    float* yr = y + row * cols;
    float m = -INFINITY, s = 0.0f;
    for (uint32_t idx = threadIdx.x; idx < nvec; idx += THREADS) {
      float f[V];
      IO::unpack(IO::load_keep(xr, idx), f);
      float lm = f[0];
#pragma unroll
      for (int j = 1; j < V; ++j) lm = fmaxf(lm, f[j]);
      if (lm > m) {  // the running max moves: rescale what was summed so far
        s *= expf(m - lm);
        m = lm;
      }
      if (m != -INFINITY) {  // nothing finite seen yet: -inf entries add 0, as in the plain formula
#pragma unroll
        for (int j = 0; j < V; ++j) s += expf(f[j] - m);
      }
    }
    const float gm = cta_allreduce<OpMax, THREADS / 32>(m, slots[0]);
    // A thread that saw nothing has m = -inf and s = 0; expf(-inf - gm) = 0 keeps it neutral
    // unless gm is -inf too (an all -inf row), which yields NaN exactly like the plain formula.
    s = (m == -INFINITY && gm != -INFINITY) ? 0.0f : s * expf(m - gm);
    const float gs = cta_allreduce<OpSum, THREADS / 32>(s, slots[1]);
    const float inv = 1.0f / gs;
    for (uint32_t idx = threadIdx.x; idx < nvec; idx += THREADS) {
      float f[V];
      IO::unpack(IO::load(xr, idx), f);
#pragma unroll
      for (int j = 0; j < V; ++j) f[j] = expf(f[j] - gm) * inv;
      IO::store(yr, idx, IO::pack(f));
    }
    __syncthreads();  // slots are rewritten by the next row
  }
}

// Long rows streamed by a cluster: the row is cut into one segment per CTA. Pass 1 streams the segment once with
// U vectors in flight per thread and keeps a running (max, sum) per thread, rescaling the sum when the max moves;
// the CTAs' (max, sum) pairs meet through distributed shared memory. Pass 2 reads the segment again -- from L2,
// where pass 1 left it: the segments in flight on the whole GPU are far smaller than L2 -- and writes y. HBM
// still sees each element once in and once out; nothing has to fit in registers, so the CTAs are small and many
// of them share an SM, each in another phase. (Requesting the next step's vectors before using the current ones
// was measured 3-6 % slower: the registers cost resident CTAs.)
__device__ __forceinline__ float ex2_approx(float v) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(v));
  return r;
}

template <int THREADS, int U>
__global__ void __launch_bounds__(THREADS)
softmax_rows_cluster_stream(const float* __restrict__ x, float* __restrict__ y, uint64_t rows, uint32_t cols, uint32_t cs,
                            uint32_t seg_vecs) {
  using IO = VecIO<float, 4>;
  __shared__ float slots[2][32];
  __shared__ float cl_max, cl_sum;  // this CTA's partials, read by the whole cluster
  const uint32_t rank = cluster_rank();
  const uint64_t row = blockIdx.x / cs;  // clusters are consecutive CTAs: one row per cluster
  // x and y are 16-byte aligned as arrays; a row whose length is not a multiple of four starts anywhere inside a
  // vector. Its first `head` and last `tail` elements (at most three each) ride with thread 0 of CTA 0, the
  // aligned vectors between them are cut into the CTAs' segments.
  const uint64_t start = row * cols;
  const uint32_t head = min(cols, (4u - static_cast<uint32_t>(start & 3u)) & 3u);
  const uint32_t nvec = (cols - head) / 4;
  const uint32_t tail = cols - head - 4 * nvec;
  const uint32_t v0 = rank * seg_vecs < nvec ? rank * seg_vecs : nvec;
  const uint32_t v1 = nvec - v0 < seg_vecs ? nvec : v0 + seg_vecs;
  const float* xe = x + start;            // the row, element-wise
  float* ye = y + start;
  const float* xr = xe + head;            // its aligned vectors
  float* yr = ye + head;
  const bool edges = rank == 0 && threadIdx.x == 0 && head + tail > 0;
  (void)rows;

  float m = -INFINITY, s = 0.0f;
  if (edges) {
    for (uint32_t j = 0; j < head + tail; ++j) m = fmaxf(m, __ldg(xe + (j < head ? j : cols - tail + (j - head))));
    if (m != -INFINITY)
      for (uint32_t j = 0; j < head + tail; ++j) s += expf(__ldg(xe + (j < head ? j : cols - tail + (j - head))) - m);
  }
  for (uint32_t base = v0 + threadIdx.x; base < v1; base += THREADS * U) {
    float f[U][4];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint32_t idx = base + u * THREADS;
      if (idx < v1) {
        IO::unpack(IO::load_keep(xr, idx), f[u]);
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) f[u][j] = -INFINITY;
      }
    }
    float lm = f[0][0];
#pragma unroll
    for (int u = 0; u < U; ++u)
#pragma unroll
      for (int j = 0; j < 4; ++j) lm = fmaxf(lm, f[u][j]);
    if (lm > m) {  // the running max moves: rescale what was summed so far
      s *= expf(m - lm);
      m = lm;
    }
    if (m != -INFINITY) {  // nothing finite seen yet: -inf entries add 0, as in the plain formula
      // The terms of the NORMALISER go through the hardware's base-2 exponential (a subtraction, a multiplication and one
      // special-function instruction instead of the ten of expf): a term is off by at most 2^-22 relative plus
      // |x - m| * 2^-24, so the sum is off by less than 3e-7 relative, below what the order of an fp32 sum of this
      // length moves it by. The outputs of pass 2 take the accurate expf like every other softmax kernel. With
      // expf here the kernel was bound by instruction issue (82 % of the issue slots at 5.4 TB/s), not by memory.
#pragma unroll
      for (int u = 0; u < U; ++u)
#pragma unroll
        for (int j = 0; j < 4; ++j) s += ex2_approx((f[u][j] - m) * 1.4426950408889634f);  // the maximum itself adds exactly 1
    }
  }
  const float cm = cta_allreduce<OpMax, THREADS / 32>(m, slots[0]);
  // A thread that saw nothing has m = -inf and s = 0; expf(-inf - cm) = 0 keeps it neutral unless cm is -inf too
  s = (m == -INFINITY && cm != -INFINITY) ? 0.0f : s * expf(m - cm);
  const float csum = cta_allreduce<OpSum, THREADS / 32>(s, slots[1]);
  if (threadIdx.x == 0) {
    cl_max = cm;
    cl_sum = csum;
  }
  cluster_sync_all();
  float gm = -INFINITY;
  for (uint32_t r = 0; r < cs; ++r) gm = fmaxf(gm, ld_dsmem(&cl_max, r));
  float gs = 0.0f;
  for (uint32_t r = 0; r < cs; ++r) {  // ascending rank: the same total in every CTA
    const float pm = ld_dsmem(&cl_max, r), ps = ld_dsmem(&cl_sum, r);
    gs += (pm == -INFINITY && gm != -INFINITY) ? 0.0f : ps * expf(pm - gm);  // an all -inf row: NaN, like the plain formula
  }
  const float inv = 1.0f / gs;
  if (edges)
    for (uint32_t j = 0; j < head + tail; ++j) {
      const uint32_t c = j < head ? j : cols - tail + (j - head);
      ye[c] = expf(__ldg(xe + c) - gm) * inv;
    }
  for (uint32_t base = v0 + threadIdx.x; base < v1; base += THREADS * U) {
    float f[U][4];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint32_t idx = base + u * THREADS;
      if (idx < v1) IO::unpack(IO::load(xr, idx), f[u]);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint32_t idx = base + u * THREADS;
      if (idx < v1) {
#pragma unroll
        for (int j = 0; j < 4; ++j) f[u][j] = expf(f[u][j] - gm) * inv;
        IO::store(yr, idx, IO::pack(f[u]));
      }
    }
  }
  cluster_sync_all();  // no CTA leaves while a peer may still read its partials
}

template <int THREADS, int U>
int launch_cluster_stream_shape(const float* x, float* y, uint64_t rows, uint32_t cols, uint32_t nvec, uint32_t cs, cudaStream_t s) {
  const uint32_t seg = (nvec + cs - 1) / cs;
  auto* fn = softmax_rows_cluster_stream<THREADS, U>;
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
  const cudaError_t e = cudaLaunchKernelEx(&cfg, fn, x, y, rows, cols, cs, seg);
  count_launch();
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(TCAB_ERR_CUDA, "softmax_rows_cluster_stream: launch failed: %s", cudaGetErrorString(e));
  }
  return TCAB_OK;
}

// Shape of the streaming clusters: 256 threads x 4 vectors per step while eight CTAs cover the row in four steps
// that way, then 512 x 4, then 512 x 8. Measured (2^27 elements, TB/s, against the register clusters
// and the shared-memory rows): 24576 columns 6.1 (5.5), 32768 5.8 (5.6), 49152 6.0 (5.1), 65536 5.5 (5.2), 98304
// 5.7 (4.9), 131072 5.3 (4.4), 262144 5.1 (4.0), 524288 4.8 (3.2), 1048576 4.3 (2.0). tune("softmax", _, p1 =
// CTAs per row, p2 = shape 1..5, p3 = 7) forces one.
int launch_cluster_stream(const float* x, float* y, uint64_t rows, uint32_t cols, uint32_t nvec, bool few_rows, cudaStream_t s) {
  const Tune& tn = tune(kSoftmax);
  uint32_t cs = 0;
  int shape = 0;
  if (tn.p3 == 7) {
    cs = tn.p1 >= 1 && tn.p1 <= 8 ? static_cast<uint32_t>(tn.p1) : 0u;
    shape = tn.p2;
  }
  if (shape <= 0 && few_rows) {  // few rows: large steps, four CTAs per row while a CTA then has at most four steps
    shape = 5;
    if (cs == 0) cs = nvec <= 65536u ? 4u : 8u;
  }
  if (shape <= 0) shape = nvec <= 8u * 1024u * 4u ? 1 : nvec <= 8u * 2048u * 4u ? 2 : 5;
  if (cs == 0) cs = stream_cluster_size(nvec, shape == 1 ? 1024u : shape == 5 ? 4096u : 2048u, true);
  switch (shape) {
    case 1: return launch_cluster_stream_shape<256, 4>(x, y, rows, cols, nvec, cs, s);
    case 2: return launch_cluster_stream_shape<512, 4>(x, y, rows, cols, nvec, cs, s);
    case 3: return launch_cluster_stream_shape<256, 8>(x, y, rows, cols, nvec, cs, s);
    case 4: return launch_cluster_stream_shape<1024, 4>(x, y, rows, cols, nvec, cs, s);
    default: return launch_cluster_stream_shape<512, 8>(x, y, rows, cols, nvec, cs, s);
  }
}

template <int TPR, int VPT, int V>
int launch_reg(const float* x, float* y, uint64_t rows, uint32_t cols, int ctas_per_sm, cudaStream_t s) {
  constexpr int THREADS = row_cta_threads(TPR);
  constexpr int GROUPS = THREADS / TPR;
  auto* fn = softmax_rows_reg<TPR, VPT, V>;
  // One CTA per group of rows, left to the hardware block scheduler: measured on B200 this beats a
  // persistent grid-stride grid (6.6 vs 5.7 TB/s at 16384 x 4096), whose CTAs move through their
  // load / reduce / store phases in lock step. A positive ctas_per_sm (tuning hook) caps the grid;
  // the kernel's row loop then takes over.
  const uint64_t need = (rows + GROUPS - 1) / GROUPS;
  uint64_t grid = ctas_per_sm > 0 ? static_cast<uint64_t>(sm_count()) * ctas_per_sm : need;
  if (grid > need) grid = need;
  if (grid > 0x7fffffffull) grid = 0x7fffffffull;
  fn<<<static_cast<unsigned>(grid), THREADS, 0, s>>>(x, y, rows, cols);
  count_launch();
  return check_launch("softmax_rows_reg");
}

// The (TPR, VPT) shapes choose_row_shape(nvec, 4) can return, plus other covers of a
// 1024-vector row that the tuning hook may select.
#define TCAB_ROW_SHAPES_BASE(X) \
  X(1, 1) X(2, 1) X(4, 1) X(8, 1) X(8, 2) X(8, 4) X(16, 4) X(32, 4) X(64, 4) X(128, 4) X(256, 4) X(512, 4) X(1024, 4) \
  X(1024, 8) X(1024, 16) X(1024, 32)
#define TCAB_ROW_SHAPES_EXTRA(X) \
  X(32, 32) X(64, 16) X(128, 8) X(512, 2) X(256, 8) X(1024, 1) \
  X(16, 5) X(32, 5) X(16, 3) X(32, 3) X(64, 3) X(128, 3) X(256, 3) X(512, 3)

}  // namespace

int launch_softmax_rows(const float* x, float* y, uint64_t rows, uint32_t cols, cudaStream_t s) {
  if (rows == 0 || cols == 0) return TCAB_OK;  // nothing to write (design/tca.md:297-299)
  const bool vec = (cols % 4 == 0) && aligned16(x) && aligned16(y);
  const uint32_t nvec = vec ? cols / 4 : cols;
  const Tune& tn = tune(kSoftmax);
  // Rows from 6144 vectors (24576 columns) up, enough of them to fill the GPU with small CTAs: streaming clusters
  // (any row length: the row ends that do not fill a vector are handled element by element).
  // With fewer rows the register clusters keep rows of up to 65536 vectors unless there are at least 32 rows of at
  // least 32768 vectors (64 x 262144: 4.1 against 2.4 TB/s; 16 x 1048576: 2.9 against 0.4 for the one-CTA kernel).
  const bool many = rows * 2 >= static_cast<uint64_t>(sm_count());
  const bool few_long = !many && (cols / 4 > 65536u || (rows >= 32 && cols / 4 >= 32768u));
  if (aligned16(x) && aligned16(y) && rows * 8 <= 0x7fffffffull && tn.p0 <= 0 &&
      (tn.p3 == 7 || (tn.p3 <= 0 && cols / 4 >= 6144u && (many || few_long))))
    return launch_cluster_stream(x, y, rows, cols, cols / 4, few_long, s);
  // rows that are not a multiple of four columns but still fit a CTA's registers as 16-byte vectors
  if (!vec && cols % 4 != 0 && cols >= 16 && aligned16(x) && aligned16(y) && tn.p0 <= 0 && tn.p3 != 6) {
    const uint32_t nv = cols / 4;  // aligned vectors inside a row, at most
    int ut = 0, uv = 0;
    if (nv <= 2048 && choose_row_shape_fit(nv, true, false, 4, &ut, &uv)) {
#define TCAB_CASE(T, P) \
  if (ut == T && uv == P) return launch_reg_unaligned<T, P>(x, y, rows, cols, s);
      TCAB_CASE(8, 1) TCAB_CASE(8, 2) TCAB_CASE(8, 4) TCAB_CASE(16, 4) TCAB_CASE(32, 4) TCAB_CASE(64, 4) TCAB_CASE(128, 4)
      TCAB_CASE(256, 4) TCAB_CASE(512, 4) TCAB_CASE(128, 8) TCAB_CASE(256, 8)
#undef TCAB_CASE
    }
    if (nv > 2048 && rows * 8 <= 0x7fffffffull) {  // clusters of 256-thread CTAs, as for aligned rows
      if (nv <= 8u * 256u * 8u && !cluster_wide(nv)) return launch_cluster_unaligned<256, 8>(x, y, rows, cols, nv, s);
      if (nv <= 8u * 256u * 16u) return launch_cluster_unaligned<256, 16>(x, y, rows, cols, nv, s);
    }
  }
  int tpr = 0, vpt = 0;
  bool fits = softmax_row_shape(nvec, vec, &tpr, &vpt);
  if (tn.p0 > 0 && tn.p1 > 0 && static_cast<uint64_t>(tn.p0) * tn.p1 >= nvec) {
    tpr = tn.p0;
    vpt = tn.p1;
    fits = true;
  }
  // Rows of 2049..11264 vectors with enough of them to fill the GPU: the shared-memory kernel (rows_smem.cu), two or
  // three CTAs per SM while the row allows it. Measured 6.0-6.3 TB/s at 10240..20480 columns (clusters: 4.8-6.1)
  // and 5.1-5.5 at 24576..45056 (clusters: 4.8-5.4). p3 == 3 forces it.
  // (30720..32768 columns: two full 16-vector CTAs per row run at 5.6-5.7, the ring of a lone CTA at 5.4-5.5)
  const bool two_full_ctas = nvec >= 7680 && nvec <= 8192 && rows * 8 <= 0x7fffffffull;
  if (vec && tn.p0 <= 0 && rows_smem_fits(static_cast<uint64_t>(cols) * 4) &&
      (tn.p3 == 3 || (tn.p3 <= 0 && nvec > 2048 && rows >= static_cast<uint64_t>(sm_count()) && !two_full_ctas)))
    return launch_softmax_rows_smem(x, y, rows, cols, s);
  // Rows beyond 2048 vectors go to the cluster kernel (2..8 CTAs of 256 threads x 8 vectors while that covers
  // the row: measured 6.1 against 4.4 TB/s for one 1024-thread CTA at 16384 columns), unless the tuning hook
  // asked for a single-CTA shape; rows beyond 8 x 8192 vectors, or more rows than the grid can index, stream.
  const bool long_class = nvec > 8u * 256u * 16u;  // 512-thread CTAs: they pay off only while the GPU is not full
  if (tn.p0 <= 0 && nvec > 2048u && nvec <= 8u * 8192u && rows * 8 <= 0x7fffffffull && tn.p3 != 1 &&
      (!long_class || rows < 2ull * sm_count() || tn.p3 == 2))
    return vec ? launch_cluster<4>(x, y, rows, cols, nvec, s) : launch_cluster<1>(x, y, rows, cols, nvec, s);
  if (fits) {
#define TCAB_CASE(T, P) \
  if (tpr == T && vpt == P) return vec ? launch_reg<T, P, 4>(x, y, rows, cols, tn.p2, s) \
                                       : launch_reg<T, P, 1>(x, y, rows, cols, tn.p2, s);
    TCAB_ROW_SHAPES_BASE(TCAB_CASE)
#undef TCAB_CASE
#define TCAB_CASE(T, P) \
  if (vec && tpr == T && vpt == P) return launch_reg<T, P, 4>(x, y, rows, cols, tn.p2, s);
    TCAB_ROW_SHAPES_EXTRA(TCAB_CASE)
#undef TCAB_CASE
    if (tn.p0 > 0) return fail(TCAB_ERR_UNSUPPORTED, "softmax: no kernel for tuned shape %d x %d", tpr, vpt);
  }
  // Long rows: one CTA per row, online pass.
  constexpr int THREADS = 512;
  const uint64_t cap = static_cast<uint64_t>(sm_count()) * 4;
  const unsigned grid = static_cast<unsigned>(rows < cap ? rows : cap);
  if (vec) {
    softmax_rows_online<THREADS, 4><<<grid, THREADS, 0, s>>>(x, y, rows, cols);
  } else {
    softmax_rows_online<THREADS, 1><<<grid, THREADS, 0, s>>>(x, y, rows, cols);
  }
  count_launch();
  return check_launch("softmax_rows_online");
}

}  // namespace tcab
