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
constexpr int kSlots = 12;
#ifndef TCAB_ROWS_SMEM_WARPS
#define TCAB_ROWS_SMEM_WARPS 16
#endif
constexpr int kConsumerWarps = TCAB_ROWS_SMEM_WARPS;
constexpr int kConsumers = 32 * kConsumerWarps;
constexpr int kThreads = kConsumers + 32;  // + the producer warp
constexpr int kSlotVecs = kSlotBytes / 16;
constexpr size_t kRingBytes = static_cast<size_t>(kSlots) * kSlotBytes;

__device__ int g_rows_smem_status = 0;

// global -> shared bulk copy of `bytes` (a multiple of 16, both addresses 16-byte aligned); completion is
// counted on `bar` in bytes.
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}

struct Ring {
  uint64_t full[kSlots];   // producer: arrive.expect_tx + the copy's bytes
  uint64_t empty[kSlots];  // one arrival per consumer warp
  float red[2][kConsumerWarps];
  int consumer_abort;      // written by consumers only, read after their barrier: a uniform decision
  int producer_abort;
};

// Sum / max over the consumer threads through shared memory; one named barrier, result in every thread.
template <typename Op>
__device__ __forceinline__ float consumers_allreduce(float v, float* slots) {
  v = warp_allreduce<Op>(v);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) slots[warp] = v;
  ptx::named_bar_sync(1, kConsumers);
  return warp_allreduce<Op>(lane < kConsumerWarps ? slots[lane] : Op::identity());
}

// The producer: every row of this CTA, slot by slot, as far ahead as the ring allows.
__device__ __forceinline__ void produce_rows(Ring& ring, uint32_t ring_base, const uint8_t* x, uint64_t rows,
                                             uint32_t row_bytes) {
  uint32_t slot = 0, phase = 0;
  volatile int* abort_p = &ring.producer_abort;
  for (uint64_t row = blockIdx.x; row < rows; row += gridDim.x) {
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

__device__ __forceinline__ void init_ring(Ring& ring) {
  if (threadIdx.x == 0) {
    for (int s = 0; s < kSlots; ++s) {
      ptx::mbar_init(ptx::smem_u32(&ring.full[s]), 1);
      ptx::mbar_init(ptx::smem_u32(&ring.empty[s]), kConsumerWarps);
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
__device__ __forceinline__ void finish_ring(Ring& ring) {
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
template <typename T, int V>
__global__ void __launch_bounds__(kThreads, 1)
layernorm_rows_smem(const T* __restrict__ x, const T* __restrict__ gamma, const T* __restrict__ beta, float eps,
                    T* __restrict__ y, uint64_t rows, uint32_t cols) {
  using IO = VecIO<T, V>;
  using Raw = typename IO::Raw;
  extern __shared__ __align__(128) uint8_t ring_mem[];
  __shared__ Ring ring;
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
    for (uint64_t row = blockIdx.x; row < rows; row += gridDim.x) {
      T* yr = y + row * cols;
      bool ok = true;
      // pass 1: the sum, slot by slot as the copies land
      float s = 0.0f;
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
#pragma unroll
            for (int i = 0; i < (kSlotVecs + kConsumers - 1) / kConsumers; ++i) {
              const uint32_t idx = threadIdx.x + i * kConsumers;
              if (idx < left && idx < static_cast<uint32_t>(kSlotVecs)) {
                float f[V];
                IO::unpack(src[idx], f);
#pragma unroll
                for (int j = 0; j < V; ++j) s += f[j];
              }
            }
          }
          if (++slot == kSlots) { slot = 0; phase ^= 1u; }
        }
      }
      const float mean = consumers_allreduce<OpSum>(s, ring.red[0]) / n;
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
      const float rstd = 1.0f / sqrtf(consumers_allreduce<OpSum>(q, ring.red[1]) / n + eps);
      // pass 3: normalise, scale, shift, store; hand each slot back once this warp has read it
      {
        uint32_t slot = slot0;
        for (uint32_t c = 0; c < nchunks; ++c) {
          const Raw* src = reinterpret_cast<const Raw*>(ring_mem + slot * kSlotBytes);
          const uint32_t left = nvec - c * kSlotVecs;
#pragma unroll
          for (int i = 0; i < (kSlotVecs + kConsumers - 1) / kConsumers; ++i) {
            const uint32_t idx = threadIdx.x + i * kConsumers;
            if (idx < left && idx < static_cast<uint32_t>(kSlotVecs)) {
              float f[V], gf[V], bf[V];
              IO::unpack(src[idx], f);
              IO::unpack(IO::load_keep(gamma, c * kSlotVecs + idx), gf);
              IO::unpack(IO::load_keep(beta, c * kSlotVecs + idx), bf);
#pragma unroll
              for (int j = 0; j < V; ++j) f[j] = (f[j] - mean) * rstd * gf[j] + bf[j];
              IO::store(yr, c * kSlotVecs + idx, IO::pack(f));
            }
          }
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&ring.empty[slot]));
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
__global__ void __launch_bounds__(kThreads, 1)
softmax_rows_smem(const float* __restrict__ x, float* __restrict__ y, uint64_t rows, uint32_t cols) {
  using IO = VecIO<float, 4>;
  extern __shared__ __align__(128) uint8_t ring_mem[];
  __shared__ Ring ring;
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
    uint32_t slot0 = 0, phase0 = 0;
    for (uint64_t row = blockIdx.x; row < rows; row += gridDim.x) {
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
      m = consumers_allreduce<OpMax>(m, ring.red[0]);
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
      const float inv = 1.0f / consumers_allreduce<OpSum>(s, ring.red[1]);
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

template <typename Fn>
int prepare(Fn* fn) {
  const cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kRingBytes));
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(TCAB_ERR_CUDA, "rows_smem: cannot reserve %zu bytes of shared memory: %s", kRingBytes, cudaGetErrorString(e));
  }
  return TCAB_OK;
}

unsigned grid_for(uint64_t rows) {
  const uint64_t sms = static_cast<uint64_t>(sm_count());
  return static_cast<unsigned>(rows < sms ? rows : sms);
}

}  // namespace

// A row fits when it leaves at least one slot of the ring free (the producer then always has room to run ahead).
bool rows_smem_fits(uint64_t row_bytes) { return row_bytes > 0 && row_bytes <= kRingBytes - kSlotBytes && row_bytes % 16 == 0; }

int rows_smem_status(int* out) {
  if (cudaMemcpyFromSymbol(out, g_rows_smem_status, sizeof(int)) != cudaSuccess) {
    cudaGetLastError();
    return fail(TCAB_ERR_CUDA, "device_status: cannot read the status word");
  }
  return TCAB_OK;
}

int launch_softmax_rows_smem(const float* x, float* y, uint64_t rows, uint32_t cols, cudaStream_t s) {
  int rc = prepare(softmax_rows_smem);
  if (rc != TCAB_OK) return rc;
  softmax_rows_smem<<<grid_for(rows), kThreads, kRingBytes, s>>>(x, y, rows, cols);
  count_launch();
  return check_launch("softmax_rows_smem");
}

int launch_layernorm_rows_smem_bf16(const __nv_bfloat16* x, const __nv_bfloat16* gamma, const __nv_bfloat16* beta,
                                    float eps, __nv_bfloat16* y, uint64_t rows, uint32_t cols, cudaStream_t s) {
  int rc = prepare(layernorm_rows_smem<__nv_bfloat16, 8>);
  if (rc != TCAB_OK) return rc;
  layernorm_rows_smem<__nv_bfloat16, 8><<<grid_for(rows), kThreads, kRingBytes, s>>>(x, gamma, beta, eps, y, rows, cols);
  count_launch();
  return check_launch("layernorm_rows_smem");
}

int launch_layernorm_rows_smem_f32(const float* x, const float* gamma, const float* beta, float eps, float* y,
                                   uint64_t rows, uint32_t cols, cudaStream_t s) {
  int rc = prepare(layernorm_rows_smem<float, 4>);
  if (rc != TCAB_OK) return rc;
  layernorm_rows_smem<float, 4><<<grid_for(rows), kThreads, kRingBytes, s>>>(x, gamma, beta, eps, y, rows, cols);
  count_launch();
  return check_launch("layernorm_rows_smem");
}

}  // namespace tcab
