// rows_smem.cu -- long rows of the map-reduce-map chains (row softmax, layer-norm) held in SHARED
// memory instead of registers.
//
// The register-resident row kernels (softmax_rows.cu, layernorm_rows.cu) keep a row in the registers of
// one CTA; beyond about 2048 vectors per row they need 512..1024-thread CTAs, few of which fit an SM, and
// the bytes in flight per SM -- what the HBM rate depends on -- fall with the occupancy (4 TB/s where short
// rows run at 6.5). Here the bytes in flight do not depend on registers at all:
//
//   * one persistent CTA per SM owns a ring of 16 KiB shared-memory slots (12 slots, 192 KiB);
//   * a producer warp (one lane) streams rows into the ring with bulk asynchronous copies
//     (cp.async.bulk global -> shared, completion counted in bytes on an mbarrier per slot), as far ahead
//     as the ring has free slots: the next row travels while the current one is reduced;
//   * sixteen consumer warps make the three passes of the chain over the slots of a row -- the reduction of
//     the first map, the reduction that needs its result (centred squares / exponentials), the final map
//     -- reading 16-byte vectors from shared memory and writing the result to global memory with
//     coalesced 16-byte stores; a slot is handed back to the producer as soon as the third pass has read it.
//
// HBM traffic is the algorithmic minimum (x once, y once); shared memory sees one write and three reads
// per byte. A row must fit the ring minus one slot (45056 fp32 / 90112 bf16 columns), rows and pointers must
// allow 16-byte vectors. Every wait on a copy or on the other role is bounded (sm100_ptx.cuh); the named
// barrier of the consumer warps is a rendezvous of warps that all walk the same rows.
#include "rowvec.cuh"
#include "sm100_ptx.cuh"

namespace tcab {
namespace {

constexpr int kSlotBytes = 16384;
constexpr int kSlotVecs = kSlotBytes / 16;

// A configuration: ring slots per CTA and consumer warps per CTA. One CTA per SM with the whole shared memory
// (12 slots, 16 warps) takes rows of up to 11 slots; rows of up to 5 (3) slots run two (three) CTAs per SM with
// 6 (4) slots and 8 consumer warps each: a CTA's passes over a row are strictly one after the other (measured:
// two barriers of 450 cycles and latency-bound chunk loops, 3,900 cycles per 32 KiB row of which the copies need
// 800), so what fills the SM is several rows in flight, not more warps on one row.
template <int SLOTS, int CW>
struct Cfg {
  static constexpr int kSlots = SLOTS;
  static constexpr int kConsumerWarps = CW;
  static constexpr int kConsumers = 32 * CW;
  static constexpr int kThreads = kConsumers + 32;  // + the producer warp
  static constexpr size_t kRingBytes = static_cast<size_t>(SLOTS) * kSlotBytes;
};

__device__ int g_rows_smem_status = 0;

// global -> shared bulk copy of `bytes` (a multiple of 16, both addresses 16-byte aligned); completion is
// counted on `bar` in bytes.
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}

template <class CF>
struct Ring {
  uint64_t full[CF::kSlots];   // producer: arrive.expect_tx + the copy's bytes
  uint64_t empty[CF::kSlots];  // one arrival per consumer warp
  float red[4][CF::kConsumerWarps];  // two reductions per row, alternating pairs from row to row
  int consumer_abort;      // written by consumers only, read after their barrier: a uniform decision
  int producer_abort;
};

// Sum / max over the consumer threads through shared memory; one named barrier, result in every thread.
template <class CF, typename Op>
__device__ __forceinline__ float consumers_allreduce(float v, float* slots) {
  v = warp_allreduce<Op>(v);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) slots[warp] = v;
  ptx::named_bar_sync(1, CF::kConsumers);
  return warp_allreduce<Op>(lane < CF::kConsumerWarps ? slots[lane] : Op::identity());
}

// Two sums at once behind ONE named barrier (each in its own slot array).
template <class CF>
__device__ __forceinline__ void consumers_allreduce2(float& a, float& b, float* slots_a, float* slots_b) {
  a = warp_allreduce<OpSum>(a);
  b = warp_allreduce<OpSum>(b);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) {
    slots_a[warp] = a;
    slots_b[warp] = b;
  }
  ptx::named_bar_sync(1, CF::kConsumers);
  a = warp_allreduce<OpSum>(lane < CF::kConsumerWarps ? slots_a[lane] : 0.0f);
  b = warp_allreduce<OpSum>(lane < CF::kConsumerWarps ? slots_b[lane] : 0.0f);
}

// The producer: every row of this CTA, slot by slot, as far ahead as the ring allows.
template <class CF>
__device__ __forceinline__ void produce_rows(Ring<CF>& ring, uint32_t ring_base, const uint8_t* x, uint64_t rows,
                                             uint32_t row_bytes) {
  constexpr int kSlots = CF::kSlots;
  uint32_t slot = 0, phase = 0;
  volatile int* abort_p = &ring.producer_abort;
  uint32_t it = 0;
  for (uint64_t row = blockIdx.x; row < rows; row += gridDim.x, ++it) {
    const uint8_t* src = x + row * row_bytes;
    for (uint32_t off = 0; off < row_bytes; off += kSlotBytes) {
      if (!ptx::mbar_wait(ptx::smem_u32(&ring.empty[slot]), phase ^ 1u, abort_p)) return;
      const uint32_t bytes = row_bytes - off < static_cast<uint32_t>(kSlotBytes) ? row_bytes - off : kSlotBytes;
      const uint32_t bar = ptx::smem_u32(&ring.full[slot]);
      ptx::mbar_expect_tx(bar, bytes);
      bulk_load(ring_base + slot * kSlotBytes, src + off, bytes, bar);
      if (++slot == kSlots) { slot = 0; phase ^= 1u; }
    }
  }
}

template <class CF>
__device__ __forceinline__ void init_ring(Ring<CF>& ring) {
  if (threadIdx.x == 0) {
    for (int s = 0; s < CF::kSlots; ++s) {
      ptx::mbar_init(ptx::smem_u32(&ring.full[s]), 1);
      ptx::mbar_init(ptx::smem_u32(&ring.empty[s]), CF::kConsumerWarps);
    }
    ring.consumer_abort = 0;
    ring.producer_abort = 0;
    ptx::fence_barrier_init();
    ptx::fence_proxy_async();
  }
  __syncthreads();
}

// What a CTA does before it exits after a wait gave up: copies may still be in flight into its shared
// memory, so it idles for a bounded time first, then records the status.
template <class CF>
__device__ __forceinline__ void finish_ring(Ring<CF>& ring) {
  __syncthreads();
  if (ring.consumer_abort != 0 || ring.producer_abort != 0) {
    const long long t0 = clock64();
    while (clock64() - t0 < 4000000ll) {
    }
    if (threadIdx.x == 0) g_rows_smem_status = 1;
  }
}

// ---------------------------------------------------------------------------------------------
// layer-norm
// ---------------------------------------------------------------------------------------------
// SHIFTED: mean and variance from ONE pass over the row, as sums of (x - K) and (x - K)^2 with K the mean of the
// row's first 32 elements (var = E[(x-K)^2] - (E[x-K])^2 cancels only when |mean - K| is large against the spread;
// a row for which it turns out to be makes the centred second pass after all). Used for bf16 rows, where unpacking is the cost of a pass and the result is rounded
// to 8 bits of mantissa; fp32 rows keep the two-pass centred variance of the register kernels and the oracle.
template <class CF, typename T, int V, bool SHIFTED, bool PF = false>
__global__ void __launch_bounds__(CF::kThreads, PF ? 12 / CF::kSlots : 1)
layernorm_rows_smem(const T* __restrict__ x, const T* __restrict__ gamma, const T* __restrict__ beta, float eps,
                    T* __restrict__ y, uint64_t rows, uint32_t cols) {
  using IO = VecIO<T, V>;
  using Raw = typename IO::Raw;
  constexpr int kSlots = CF::kSlots, kConsumers = CF::kConsumers;
  extern __shared__ __align__(128) uint8_t ring_mem[];
  __shared__ Ring<CF> ring;
  init_ring(ring);
  const uint32_t ring_base = ptx::smem_u32(ring_mem);
  const uint32_t row_bytes = cols * static_cast<uint32_t>(sizeof(T));
  const uint32_t nchunks = (row_bytes + kSlotBytes - 1) / kSlotBytes;
  const uint32_t nvec = cols / V;
  const float n = static_cast<float>(cols);

  if (threadIdx.x >= kConsumers) {
    if (threadIdx.x == kConsumers) produce_rows(ring, ring_base, reinterpret_cast<const uint8_t*>(x), rows, row_bytes);
  } else {
    volatile int* abort_p = &ring.consumer_abort;
    const int lane = threadIdx.x & 31;
    uint32_t slot0 = 0, phase0 = 0;  // ring position of the row's first slot
    uint32_t it = 0;
    for (uint64_t row = blockIdx.x; row < rows; row += gridDim.x, ++it) {
      // the slot arrays of this row's reductions: the other pair than the previous row's, so that a warp that runs
      // ahead into the next row never overwrites what a slower warp has yet to read
      float* red_a = ring.red[2 * (it & 1u)];
      float* red_b = ring.red[2 * (it & 1u) + 1];
      T* yr = y + row * cols;
      bool ok = true;
      // pass 1: the sum (SHIFTED: of x - K, and of its square), slot by slot as the copies land
      float s = 0.0f, s2 = 0.0f, shift = 0.0f;
      {
        uint32_t slot = slot0, phase = phase0;
        for (uint32_t c = 0; c < nchunks; ++c) {
          if (ok && !ptx::mbar_wait(ptx::smem_u32(&ring.full[slot]), phase, abort_p)) {
            ok = false;
            ring.consumer_abort = 1;
          }
          if (ok) {
            const Raw* src = reinterpret_cast<const Raw*>(ring_mem + slot * kSlotBytes);
            const uint32_t left = nvec - c * kSlotVecs;
            if (SHIFTED && c == 0) {  // every thread reads the row's first vectors (broadcasts): K = their mean
              const uint32_t kv = left < 4u ? left : 4u;
              float acc = 0.0f;
              for (uint32_t q = 0; q < kv; ++q) {
                float f0[V];
                IO::unpack(src[q], f0);
#pragma unroll
                for (int j = 0; j < V; ++j) acc += f0[j];
              }
              shift = acc / static_cast<float>(kv * V);
            }
#pragma unroll
            for (int i = 0; i < (kSlotVecs + kConsumers - 1) / kConsumers; ++i) {
              const uint32_t idx = threadIdx.x + i * kConsumers;
              if (idx < left && idx < static_cast<uint32_t>(kSlotVecs)) {
                float f[V];
                IO::unpack(src[idx], f);
#pragma unroll
                for (int j = 0; j < V; ++j) {
                  if (SHIFTED) {
                    const float d = f[j] - shift;
                    s += d;
                    s2 += d * d;
                  } else {
                    s += f[j];
                  }
                }
              }
            }
          }
          if (++slot == kSlots) { slot = 0; phase ^= 1u; }
        }
      }
      // PF: gamma and beta of a slot are loaded one slot ahead (those of the first slot here, before the
      // reductions), so that their trip from L2 is not paid between a slot's hand-back and the next slot's work:
      // with the ring taking most of the SM's L1 they come from L2 for every row. Measured: fp32 16384 / 20480
      // columns 4.8 / 5.0 -> 5.6 TB/s, rows of one CTA per SM +2-6 %. The second register set does not fit three
      // CTAs per SM (it spills there: 5.7 -> 4.0 TB/s), so that shape keeps the loads in the third pass.
      constexpr int kIter = (kSlotVecs + kConsumers - 1) / kConsumers;
      Raw gcur[PF ? kIter : 1] = {}, bcur[PF ? kIter : 1] = {};
      auto load_params = [&](uint32_t c, Raw* gq, Raw* bq) {
        const uint32_t left = nvec - c * kSlotVecs;
#pragma unroll
        for (int i = 0; i < kIter; ++i) {
          const uint32_t idx = threadIdx.x + i * kConsumers;
          if (idx < left && idx < static_cast<uint32_t>(kSlotVecs)) {
            gq[i] = IO::load_keep(gamma, c * kSlotVecs + idx);
            bq[i] = IO::load_keep(beta, c * kSlotVecs + idx);
          }
        }
      };
      if constexpr (PF) load_params(0, gcur, bcur);
      float mean, rstd;
      if (SHIFTED) {
        float d1 = s, d2 = s2;
        consumers_allreduce2<CF>(d1, d2, red_a, red_b);
        if (ring.consumer_abort != 0) break;  // uniform: written before the barrier above, by consumers only
        const float m1 = d1 / n;
        mean = shift + m1;
        const float var = fmaxf(d2 / n - m1 * m1, 0.0f);
        rstd = 1.0f / sqrtf(var + eps);
        if (m1 * m1 > var) {
          // K was a poor guess of the mean (further from it than one standard deviation): the difference above has
          // cancelled digits, so this row takes the centred second pass after all. The test is on reduced values:
          // every consumer thread decides the same way.
          float q = 0.0f;
          uint32_t slot = slot0;
          for (uint32_t c = 0; c < nchunks; ++c) {
            const Raw* src = reinterpret_cast<const Raw*>(ring_mem + slot * kSlotBytes);
            const uint32_t left = nvec - c * kSlotVecs;
#pragma unroll
            for (int i = 0; i < (kSlotVecs + kConsumers - 1) / kConsumers; ++i) {
              const uint32_t idx = threadIdx.x + i * kConsumers;
              if (idx < left && idx < static_cast<uint32_t>(kSlotVecs)) {
                float f[V];
                IO::unpack(src[idx], f);
#pragma unroll
                for (int j = 0; j < V; ++j) q += (f[j] - mean) * (f[j] - mean);
              }
            }
            if (++slot == kSlots) slot = 0;
          }
          ptx::named_bar_sync(1, CF::kConsumers);  // every warp has read the first reduction's slots
          float unused = 0.0f;
          consumers_allreduce2<CF>(q, unused, red_a, red_b);
          rstd = 1.0f / sqrtf(q / n + eps);
        }
      } else {
      mean = consumers_allreduce<CF, OpSum>(s, red_a) / n;
      if (ring.consumer_abort != 0) break;  // uniform: written before the barrier above, by consumers only
      // pass 2: centred squares
      float q = 0.0f;
      {
        uint32_t slot = slot0;
        for (uint32_t c = 0; c < nchunks; ++c) {
          const Raw* src = reinterpret_cast<const Raw*>(ring_mem + slot * kSlotBytes);
          const uint32_t left = nvec - c * kSlotVecs;
#pragma unroll
          for (int i = 0; i < (kSlotVecs + kConsumers - 1) / kConsumers; ++i) {
            const uint32_t idx = threadIdx.x + i * kConsumers;
            if (idx < left && idx < static_cast<uint32_t>(kSlotVecs)) {
              float f[V];
              IO::unpack(src[idx], f);
#pragma unroll
              for (int j = 0; j < V; ++j) q += (f[j] - mean) * (f[j] - mean);
            }
          }
          if (++slot == kSlots) slot = 0;
        }
      }
      rstd = 1.0f / sqrtf(consumers_allreduce<CF, OpSum>(q, red_b) / n + eps);
      }
      // pass 3: normalise, scale, shift, store; hand each slot back once this warp has read it
      {
        uint32_t slot = slot0;
        for (uint32_t c = 0; c < nchunks; ++c) {
          const Raw* src = reinterpret_cast<const Raw*>(ring_mem + slot * kSlotBytes);
          const uint32_t left = nvec - c * kSlotVecs;
          Raw gnext[PF ? kIter : 1] = {}, bnext[PF ? kIter : 1] = {};
          if constexpr (PF) {
            if (c + 1 < nchunks) load_params(c + 1, gnext, bnext);
          }
#pragma unroll
          for (int i = 0; i < kIter; ++i) {
            const uint32_t idx = threadIdx.x + i * kConsumers;
            if (idx < left && idx < static_cast<uint32_t>(kSlotVecs)) {
              float f[V], gf[V], bf[V];
              IO::unpack(src[idx], f);
              if constexpr (PF) {
                IO::unpack(gcur[i], gf);
                IO::unpack(bcur[i], bf);
              } else {
                IO::unpack(IO::load_keep(gamma, c * kSlotVecs + idx), gf);
                IO::unpack(IO::load_keep(beta, c * kSlotVecs + idx), bf);
              }
#pragma unroll
              for (int j = 0; j < V; ++j) f[j] = (f[j] - mean) * rstd * gf[j] + bf[j];
              IO::store(yr, c * kSlotVecs + idx, IO::pack(f));
            }
          }
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&ring.empty[slot]));
          if constexpr (PF) {
#pragma unroll
            for (int i = 0; i < kIter; ++i) {
              gcur[i] = gnext[i];
              bcur[i] = bnext[i];
            }
          }
          if (++slot == kSlots) slot = 0;
        }
      }
      // the next row starts where this one ended
      slot0 += nchunks;
      while (slot0 >= static_cast<uint32_t>(kSlots)) { slot0 -= kSlots; phase0 ^= 1u; }
    }
  }
  finish_ring(ring);
}

// ---------------------------------------------------------------------------------------------
// row softmax
// ---------------------------------------------------------------------------------------------
template <class CF>
__global__ void __launch_bounds__(CF::kThreads, 1)
softmax_rows_smem(const float* __restrict__ x, float* __restrict__ y, uint64_t rows, uint32_t cols) {
  using IO = VecIO<float, 4>;
  constexpr int kSlots = CF::kSlots, kConsumers = CF::kConsumers;
  extern __shared__ __align__(128) uint8_t ring_mem[];
  __shared__ Ring<CF> ring;
  init_ring(ring);
  const uint32_t ring_base = ptx::smem_u32(ring_mem);
  const uint32_t row_bytes = cols * 4u;
  const uint32_t nchunks = (row_bytes + kSlotBytes - 1) / kSlotBytes;
  const uint32_t nvec = cols / 4;

  if (threadIdx.x >= kConsumers) {
    if (threadIdx.x == kConsumers) produce_rows(ring, ring_base, reinterpret_cast<const uint8_t*>(x), rows, row_bytes);
  } else {
    volatile int* abort_p = &ring.consumer_abort;
    const int lane = threadIdx.x & 31;
    uint32_t slot0 = 0, phase0 = 0, it = 0;
    for (uint64_t row = blockIdx.x; row < rows; row += gridDim.x, ++it) {
      float* yr = y + row * cols;
      bool ok = true;
      float m = -INFINITY;
      {
        uint32_t slot = slot0, phase = phase0;
        for (uint32_t c = 0; c < nchunks; ++c) {
          if (ok && !ptx::mbar_wait(ptx::smem_u32(&ring.full[slot]), phase, abort_p)) {
            ok = false;
            ring.consumer_abort = 1;
          }
          if (ok) {
            const float4* src = reinterpret_cast<const float4*>(ring_mem + slot * kSlotBytes);
            const uint32_t left = nvec - c * kSlotVecs;
#pragma unroll
            for (int i = 0; i < (kSlotVecs + kConsumers - 1) / kConsumers; ++i) {
              const uint32_t idx = threadIdx.x + i * kConsumers;
              if (idx < left && idx < static_cast<uint32_t>(kSlotVecs)) {
                const float4 f = src[idx];
                m = fmaxf(fmaxf(m, fmaxf(f.x, f.y)), fmaxf(f.z, f.w));
              }
            }
          }
          if (++slot == kSlots) { slot = 0; phase ^= 1u; }
        }
      }
      m = consumers_allreduce<CF, OpMax>(m, ring.red[0]);
      if (ring.consumer_abort != 0) break;
      // pass 2: the exponentials are kept (written back to the slot), so that pass 3 only scales them
      float s = 0.0f;
      {
        uint32_t slot = slot0;
        for (uint32_t c = 0; c < nchunks; ++c) {
          float4* src = reinterpret_cast<float4*>(ring_mem + slot * kSlotBytes);
          const uint32_t left = nvec - c * kSlotVecs;
#pragma unroll
          for (int i = 0; i < (kSlotVecs + kConsumers - 1) / kConsumers; ++i) {
            const uint32_t idx = threadIdx.x + i * kConsumers;
            if (idx < left && idx < static_cast<uint32_t>(kSlotVecs)) {
              float4 f = src[idx];
              f.x = expf(f.x - m); f.y = expf(f.y - m); f.z = expf(f.z - m); f.w = expf(f.w - m);
              s += f.x; s += f.y; s += f.z; s += f.w;
              src[idx] = f;  // the same thread reads it back in pass 3
            }
          }
          if (++slot == kSlots) slot = 0;
        }
      }
      const float inv = 1.0f / consumers_allreduce<CF, OpSum>(s, ring.red[1]);
      {
        uint32_t slot = slot0;
        for (uint32_t c = 0; c < nchunks; ++c) {
          const float4* src = reinterpret_cast<const float4*>(ring_mem + slot * kSlotBytes);
          const uint32_t left = nvec - c * kSlotVecs;
#pragma unroll
          for (int i = 0; i < (kSlotVecs + kConsumers - 1) / kConsumers; ++i) {
            const uint32_t idx = threadIdx.x + i * kConsumers;
            if (idx < left && idx < static_cast<uint32_t>(kSlotVecs)) {
              float4 f = src[idx];
              float o[4] = {f.x * inv, f.y * inv, f.z * inv, f.w * inv};
              IO::store(yr, c * kSlotVecs + idx, IO::pack(o));
            }
          }
          // the slot was written by generic stores (pass 2): every thread orders its own before the next
          // bulk copy into the slot, then the warp meets, then one lane hands the slot back
          ptx::fence_proxy_async();
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&ring.empty[slot]));
          if (++slot == kSlots) slot = 0;
        }
      }
      slot0 += nchunks;
      while (slot0 >= static_cast<uint32_t>(kSlots)) { slot0 -= kSlots; phase0 ^= 1u; }
    }
  }
  finish_ring(ring);
}

// The three configurations: CTAs per SM x ring slots x consumer warps.
typedef Cfg<12, 16> Whole;   // 1 CTA per SM, rows of up to 11 slots
typedef Cfg<6, 8> Half;      // 2 CTAs per SM, rows of up to 5 slots
typedef Cfg<4, 8> Third;     // 3 CTAs per SM, rows of up to 3 slots

template <class CF, typename Fn, typename... Args>
int launch_cfg(Fn* fn, int ctas_per_sm, uint64_t rows, cudaStream_t s, const char* what, Args... args) {
  const cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(CF::kRingBytes));
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(TCAB_ERR_CUDA, "rows_smem: cannot reserve %zu bytes of shared memory: %s", CF::kRingBytes,
                cudaGetErrorString(e));
  }
  const uint64_t resident = static_cast<uint64_t>(sm_count()) * ctas_per_sm;
  const unsigned grid = static_cast<unsigned>(rows < resident ? rows : resident);
  fn<<<grid, CF::kThreads, CF::kRingBytes, s>>>(args...);
  count_launch();
  return check_launch(what);
}

// 0: one CTA per SM, 1: two, 2: three -- the most CTAs whose ring still holds a row plus one free slot.
// tune("softmax" / "layernorm", _, _, p2 = 1 | 2 | 3) forces the number of CTAs per SM where the row allows it.
int pick_cfg(uint64_t row_bytes, int forced_ctas) {
  const uint64_t slots = (row_bytes + kSlotBytes - 1) / kSlotBytes;
  int best = slots <= 3 ? 2 : slots <= 5 ? 1 : 0;
  if (forced_ctas >= 1 && forced_ctas <= 3 && forced_ctas - 1 <= best) best = forced_ctas - 1;
  return best;
}

}  // namespace

// A row fits when it leaves at least one slot of the largest ring free (the producer then always has room to
// run ahead).
bool rows_smem_fits(uint64_t row_bytes) {
  return row_bytes > 0 && row_bytes <= Whole::kRingBytes - kSlotBytes && row_bytes % 16 == 0;
}

int rows_smem_status(int* out) {
  if (cudaMemcpyFromSymbol(out, g_rows_smem_status, sizeof(int)) != cudaSuccess) {
    cudaGetLastError();
    return fail(TCAB_ERR_CUDA, "device_status: cannot read the status word");
  }
  return TCAB_OK;
}

int launch_softmax_rows_smem(const float* x, float* y, uint64_t rows, uint32_t cols, cudaStream_t s) {
  switch (pick_cfg(static_cast<uint64_t>(cols) * 4, tune(kSoftmax).p2)) {
    case 2: return launch_cfg<Third>(softmax_rows_smem<Third>, 3, rows, s, "softmax_rows_smem", x, y, rows, cols);
    case 1: return launch_cfg<Half>(softmax_rows_smem<Half>, 2, rows, s, "softmax_rows_smem", x, y, rows, cols);
    default: return launch_cfg<Whole>(softmax_rows_smem<Whole>, 1, rows, s, "softmax_rows_smem", x, y, rows, cols);
  }
}

int launch_layernorm_rows_smem_bf16(const __nv_bfloat16* x, const __nv_bfloat16* gamma, const __nv_bfloat16* beta,
                                    float eps, __nv_bfloat16* y, uint64_t rows, uint32_t cols, cudaStream_t s) {
  typedef __nv_bfloat16 B;
  const bool pf = tune(kLayernorm).p1 != 8;  // p1 == 8: no gamma / beta prefetch (for comparisons)
  switch (pick_cfg(static_cast<uint64_t>(cols) * 2, tune(kLayernorm).p2)) {
    case 2: return launch_cfg<Third>(layernorm_rows_smem<Third, B, 8, true>, 3, rows, s, "layernorm_rows_smem", x, gamma, beta, eps, y, rows, cols);
    case 1:
      if (pf) return launch_cfg<Half>(layernorm_rows_smem<Half, B, 8, true, true>, 2, rows, s, "layernorm_rows_smem", x, gamma, beta, eps, y, rows, cols);
      return launch_cfg<Half>(layernorm_rows_smem<Half, B, 8, true>, 2, rows, s, "layernorm_rows_smem", x, gamma, beta, eps, y, rows, cols);
    default:
      if (pf) return launch_cfg<Whole>(layernorm_rows_smem<Whole, B, 8, true, true>, 1, rows, s, "layernorm_rows_smem", x, gamma, beta, eps, y, rows, cols);
      return launch_cfg<Whole>(layernorm_rows_smem<Whole, B, 8, true>, 1, rows, s, "layernorm_rows_smem", x, gamma, beta, eps, y, rows, cols);
  }
}

int launch_layernorm_rows_smem_f32(const float* x, const float* gamma, const float* beta, float eps, float* y,
                                   uint64_t rows, uint32_t cols, cudaStream_t s) {
  const bool pf = tune(kLayernorm).p1 != 8;
  switch (pick_cfg(static_cast<uint64_t>(cols) * 4, tune(kLayernorm).p2)) {
    case 2: return launch_cfg<Third>(layernorm_rows_smem<Third, float, 4, false>, 3, rows, s, "layernorm_rows_smem", x, gamma, beta, eps, y, rows, cols);
    case 1:
      if (pf) return launch_cfg<Half>(layernorm_rows_smem<Half, float, 4, false, true>, 2, rows, s, "layernorm_rows_smem", x, gamma, beta, eps, y, rows, cols);
      return launch_cfg<Half>(layernorm_rows_smem<Half, float, 4, false>, 2, rows, s, "layernorm_rows_smem", x, gamma, beta, eps, y, rows, cols);
    default:
      if (pf) return launch_cfg<Whole>(layernorm_rows_smem<Whole, float, 4, false, true>, 1, rows, s, "layernorm_rows_smem", x, gamma, beta, eps, y, rows, cols);
      return launch_cfg<Whole>(layernorm_rows_smem<Whole, float, 4, false>, 1, rows, s, "layernorm_rows_smem", x, gamma, beta, eps, y, rows, cols);
  }
}

}  // namespace tcab
