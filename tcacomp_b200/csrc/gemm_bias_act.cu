// gemm_bias_act.cu -- tiled bf16 contraction with a fused epilogue on the 5th-generation
// tensor cores: c = act(a @ b + bias), fp32 accumulation in TMEM, bf16 result.
//
// The reference emits a GEMM that produces ONE output element per CTA bracket with a
// K split over warps and scalar FMAs (the suite's testing/kernels/llm/gemm.tca, runner
// testing/runners/gemm.cu:44-56) and cannot bind the bias operand of the piped map
// (design/RELEASE-v0.0.0.md:150). Here:
//
//   * a persistent CTA per SM walks 256x256 output tiles; K is cut into 64-wide blocks;
//   * warp 0 (one lane) is the TMA producer: per K block it loads a 256x64 slab of A
//     (K-major, rows of 128 bytes) and four 64x64 boxes of B (b is [K,N] row-major, i.e.
//     N-major: each box is 64 k-rows of 64 contiguous n) into a 3-stage shared-memory ring,
//     all with the 128-byte swizzle the tensor core expects;
//   * warp 1 (one lane) issues tcgen05.mma (M=128, N=256, K=16) into two TMEM accumulators
//     (rows 0-127 and 128-255 of the tile, 256 fp32 columns each = all 512 TMEM columns),
//     frees a ring stage with tcgen05.commit, and signals the epilogue per tile;
//   * warps 2-9 are the epilogue. The K loop runs at the tensor pipe's rate; what costs time is how long
//     the next tile's first MMAs wait for the accumulators, so the drain hands TMEM back first: each warp
//     pulls its 128 columns of accumulator 0 into registers (four tcgen05.ld of 32 lanes x 32 columns),
//     arrives on the accumulator's barrier, and only then adds the bias (staged in shared memory while
//     the K loop ran), applies the activation, rounds to bf16 and stages 32-row x 32-column half boxes in
//     two alternating shared-memory buffers (64-byte swizzle, conflict-free 16-byte stores) for TMA
//     stores, which write 64-byte row segments and clip ragged edges. Register blocks that have been
//     staged are refilled from accumulator 1, which is handed back after the fourth half box.
//
// Per K block a CTA moves 64 KB into shared memory for 8.4 MFLOP (131 flop per byte), which
// is what lets one CTA per SM run without cluster multicast. Every wait on another agent (TMA,
// tensor core, another role's arrival) is bounded (see sm100_ptx.cuh); a wait that gives up makes the
// kernel write a status word and return. The epilogue's named barrier is a rendezvous of warps that
// all walk the same tile list and never leave it early, also after a wait has given up.
#include <cuda.h>

#include <map>
#include <mutex>
#include <utility>

#include "common.cuh"
#include "sm100_ptx.cuh"

namespace tcab {
namespace {

constexpr int BM = 256, BN = 256, BK = 64;
constexpr int UMMA_M = 128, UMMA_N = 256, UMMA_K = 16;
constexpr int STAGES = 3;
constexpr int A_STAGE_BYTES = BM * BK * 2;  // 32 KB: 256 rows x 128 B
constexpr int B_STAGE_BYTES = BK * BN * 2;  // 32 KB: 4 atoms x (64 k-rows x 128 B)
constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr int B_ATOM_BYTES = BK * 128;      // one 64(n) x 64(k) box
constexpr int EPI_WARPS = 8;
constexpr int THREADS = 64 + 32 * EPI_WARPS;
constexpr int TMEM_COLS = 512;
constexpr int EPI_BOX_BYTES = 32 * 128;     // one warp's staging box: 32 rows x 64 bf16
constexpr size_t SMEM_BYTES =
    static_cast<size_t>(STAGES) * STAGE_BYTES + EPI_WARPS * EPI_BOX_BYTES + 1024;  // + alignment slack

// Device status of the last contraction kernel that gave up on a wait (0 = none).
__device__ int g_gemm_status = 0;

struct TileCoord {
  uint32_t m, n;
};
// Tiles are walked in bands of 8 tile-rows so that the CTAs running at the same time share
// A slabs and B slabs in L2.
__device__ __forceinline__ TileCoord tile_coord(uint32_t t, uint32_t tiles_m, uint32_t tiles_n) {
  const uint32_t band = 8 * tiles_n;
  const uint32_t first_m = (t / band) * 8;
  const uint32_t rows = min(8u, tiles_m - first_m);
  const uint32_t r = t % band;
  return {first_m + r % rows, r / rows};
}

// The bias of a tile, held across a warp: lane l keeps the four values of columns 4l..4l+3 of the
// warp's 128 columns. Loaded once per tile BEFORE the wait for the accumulator, so the latency of the
// global load hides under the K loop; a load inside the drain would sit on the critical path (the asm
// statements around it keep the compiler from hoisting it).
struct BiasRegs {
  float v[4];
};
__device__ __forceinline__ BiasRegs load_bias_regs(const float* __restrict__ bias, bool bias_vec, uint32_t col, uint32_t N) {
  BiasRegs b = {{0.0f, 0.0f, 0.0f, 0.0f}};
  if (bias != nullptr && col < N) {  // N % 8 == 0 and col % 4 == 0: the four columns are inside together
    if (bias_vec) {
      const float4 q = __ldg(reinterpret_cast<const float4*>(bias + col));
      b.v[0] = q.x; b.v[1] = q.y; b.v[2] = q.z; b.v[3] = q.w;
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) b.v[j] = __ldg(bias + col + j);
    }
  }
  return b;
}

// One 32-row x 64-column box of the result: TMEM -> registers -> bias / activation -> bf16 ->
// this warp's swizzled staging box. `cbase` is the box's first column within the warp's 128 columns.
__device__ __forceinline__ void stage_box_from_tmem(uint32_t taddr, bool have_acc, const BiasRegs& bias, uint32_t cbase,
                                                    int act, uint32_t my_row, int lane) {
#pragma unroll
  for (uint32_t h = 0; h < 2; ++h) {
    uint32_t r[32];
    if (have_acc) {
      ptx::tmem_ld_32x32(taddr + h * 32, r);
      ptx::tmem_ld_wait();
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j) r[j] = 0u;  // empty reduction: the accumulator's init
    }
#pragma unroll
    for (int v = 0; v < 4; ++v) {  // four 16-byte chunks of 8 columns
      const int src_lane = static_cast<int>((cbase + h * 32 + v * 8) >> 2);
      uint32_t w[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float f0 = __uint_as_float(r[v * 8 + 2 * j]) + __shfl_sync(0xffffffffu, bias.v[(2 * j) & 3], src_lane + (j >> 1));
        float f1 = __uint_as_float(r[v * 8 + 2 * j + 1]) + __shfl_sync(0xffffffffu, bias.v[(2 * j + 1) & 3], src_lane + (j >> 1));
        if (act == TCAB_ACT_RELU) {
          f0 = fmaxf(f0, 0.0f);
          f1 = fmaxf(f1, 0.0f);
        }
        const __nv_bfloat162 hh = __floats2bfloat162_rn(f0, f1);
        w[j] = *reinterpret_cast<const uint32_t*>(&hh);
      }
      // 128-byte swizzle: 16-byte chunk c of row r lives at chunk position c ^ (r % 8)
      const uint32_t chunk = (h * 4 + v) ^ (static_cast<uint32_t>(lane) & 7u);
      ptx::st_shared_v4(my_row + chunk * 16, w[0], w[1], w[2], w[3]);
    }
  }
}

// Half a box (32 rows x 32 columns) from registers: bias / activation -> bf16 -> a 2 KB staging buffer
// with 64-byte rows and the 64-byte swizzle (16-byte chunk c of row r at chunk position c ^ ((r / 2) % 4)),
// which keeps the 16-byte stores of a warp conflict-free. `bias32` points at the 32 bias values of these
// columns in shared memory; every lane reads the same addresses (broadcast).
__device__ __forceinline__ void stage_half_box(const uint32_t (&r)[32], const float* bias32, int act, uint32_t buf,
                                               int lane) {
  const uint32_t my_row = buf + static_cast<uint32_t>(lane) * 64u;
  const uint32_t sw = (static_cast<uint32_t>(lane) >> 1) & 3u;
  uint32_t w[16];
  // all the arithmetic first, then the stores: the store statements are compiler barriers, and one per
  // chunk in between would chain the four chunks' shared-memory loads one after the other
#pragma unroll
  for (int v = 0; v < 4; ++v) {  // four 16-byte chunks of 8 columns
    const float4 b0 = *reinterpret_cast<const float4*>(bias32 + v * 8);
    const float4 b1 = *reinterpret_cast<const float4*>(bias32 + v * 8 + 4);
    const float bv[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float f0 = __uint_as_float(r[v * 8 + 2 * j]) + bv[2 * j];
      const float f1 = __uint_as_float(r[v * 8 + 2 * j + 1]) + bv[2 * j + 1];
      __nv_bfloat162 hh = __floats2bfloat162_rn(f0, f1);
      // max(round(x), 0) == round(max(x, 0)): rounding keeps the sign, so the activation runs on the packed pair
      if (act == TCAB_ACT_RELU) hh = __hmax2(hh, __floats2bfloat162_rn(0.0f, 0.0f));
      w[v * 4 + j] = *reinterpret_cast<const uint32_t*>(&hh);
    }
  }
#pragma unroll
  for (int v = 0; v < 4; ++v)
    ptx::st_shared_v4(my_row + ((static_cast<uint32_t>(v) ^ sw) * 16u), w[v * 4], w[v * 4 + 1], w[v * 4 + 2], w[v * 4 + 3]);
}

// The same half box as fp32 for the contraction chains that store what they accumulate: 32 rows x 32 columns,
// scaled, to a 4 KB staging buffer with 128-byte rows and the 128-byte swizzle (chunk c of row r at c ^ (r % 8)).
__device__ __forceinline__ void stage_half_box_f32(const uint32_t (&r)[32], float alpha, uint32_t buf, int lane) {
  const uint32_t my_row = buf + static_cast<uint32_t>(lane) * 128u;
  const uint32_t sw = static_cast<uint32_t>(lane) & 7u;
#pragma unroll
  for (uint32_t v = 0; v < 8; ++v)
    ptx::st_shared_v4(my_row + ((v ^ sw) * 16u), __float_as_uint(__uint_as_float(r[v * 4]) * alpha),
                      __float_as_uint(__uint_as_float(r[v * 4 + 1]) * alpha), __float_as_uint(__uint_as_float(r[v * 4 + 2]) * alpha),
                      __float_as_uint(__uint_as_float(r[v * 4 + 3]) * alpha));
}

// OUT_F32: c is fp32 and receives alpha * accumulator (no bias, no activation): the tensor-core form of a
// contraction chain over bf16 operands whose map is the plain product. B_NK: b is [N, K] (K contiguous) instead of
// [K, N]; its tile is then K-major in shared memory like a's.
template <bool OUT_F32, bool B_NK>
__global__ void __launch_bounds__(THREADS, 1)
gemm_bias_act_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                     const __grid_constant__ CUtensorMap tmap_c, const float* __restrict__ bias, uint32_t M,
                     uint32_t N, uint32_t K, int act, float alpha) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_full[STAGES];
  __shared__ __align__(8) uint64_t bar_empty[STAGES];
  __shared__ __align__(8) uint64_t bar_tmem_full;
  __shared__ __align__(8) uint64_t bar_tmem_empty[2];
  __shared__ __align__(16) float bias_s[BN];  // the current tile's bias (zeros past N or without a bias)
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;  // the swizzle needs 1024-byte tiles
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int* abort_p = &abort_flag;

  const uint32_t tiles_m = (M + BM - 1) / BM, tiles_n = (N + BN - 1) / BN;
  const uint32_t num_tiles = tiles_m * tiles_n;
  const uint32_t num_kb = (K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) {
      ptx::mbar_init(ptx::smem_u32(&bar_full[s]), 1);
      ptx::mbar_init(ptx::smem_u32(&bar_empty[s]), 1);
    }
    ptx::mbar_init(ptx::smem_u32(&bar_tmem_full), 1);
    ptx::mbar_init(ptx::smem_u32(&bar_tmem_empty[0]), EPI_WARPS);
    ptx::mbar_init(ptx::smem_u32(&bar_tmem_empty[1]), EPI_WARPS);
    ptx::fence_barrier_init();
    ptx::fence_proxy_async();
    ptx::prefetch_tensormap(&tmap_a);
    ptx::prefetch_tensormap(&tmap_b);
    ptx::prefetch_tensormap(&tmap_c);
  }
  if (warp == 1) {
    ptx::tmem_alloc(ptx::smem_u32(&tmem_base_slot), TMEM_COLS);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (uint32_t t = blockIdx.x; ok && t < num_tiles; t += gridDim.x) {
        const TileCoord tc = tile_coord(t, tiles_m, tiles_n);
        for (uint32_t kb = 0; kb < num_kb; ++kb) {
          if (!ptx::mbar_wait(ptx::smem_u32(&bar_empty[stage]), phase ^ 1u, abort_p)) { ok = false; break; }
          const uint32_t full = ptx::smem_u32(&bar_full[stage]);
          const uint32_t a_dst = smem_base + stage * STAGE_BYTES;
          const uint32_t b_dst = a_dst + A_STAGE_BYTES;
          ptx::mbar_expect_tx(full, STAGE_BYTES);
          ptx::tma_load_2d(a_dst, &tmap_a, full, static_cast<int32_t>(kb * BK), static_cast<int32_t>(tc.m * BM));
          if (B_NK) {  // one box: 256 rows of n, 64 of k
            ptx::tma_load_2d(b_dst, &tmap_b, full, static_cast<int32_t>(kb * BK), static_cast<int32_t>(tc.n * BN));
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              ptx::tma_load_2d(b_dst + j * B_ATOM_BYTES, &tmap_b, full, static_cast<int32_t>(tc.n * BN + j * 64),
                               static_cast<int32_t>(kb * BK));
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t idesc = ptx::idesc_bf16_f32(UMMA_M, UMMA_N, /*a_mn=*/0, /*b_mn=*/B_NK ? 0 : 1);
      uint32_t stage = 0, phase = 0, tile_iter = 0;
      bool ok = true;
      for (uint32_t t = blockIdx.x; ok && t < num_tiles; t += gridDim.x, ++tile_iter) {
        for (uint32_t kb = 0; ok && kb < num_kb; ++kb) {
          if (!ptx::mbar_wait(ptx::smem_u32(&bar_full[stage]), phase, abort_p)) { ok = false; break; }
          ptx::tc_fence_after();
          const uint32_t a_src = smem_base + stage * STAGE_BYTES;
          const uint32_t b_src = a_src + A_STAGE_BYTES;
#pragma unroll
          for (int a = 0; a < 2; ++a) {
            if (kb == 0) {  // the epilogue must have drained this accumulator (previous tile)
              if (!ptx::mbar_wait(ptx::smem_u32(&bar_tmem_empty[a]), (tile_iter & 1u) ^ 1u, abort_p)) { ok = false; break; }
              ptx::tc_fence_after();
            }
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k) {
              // A: K-major, 8-row groups 1024 B apart; one UMMA_K step is 32 B inside the 128-B swizzle row.
              const uint64_t adesc = ptx::smem_desc_sw128(a_src + a * (UMMA_M * 128) + k * (UMMA_K * 2), 16, 1024);
              // B: N-major, 64-wide n atoms B_ATOM_BYTES apart, 8-k-row groups 1024 B apart; one step is 16 k-rows.
              // ([N, K] operand: K-major like A, 256 rows of n in 8-row groups 1024 B apart)
              const uint64_t bdesc = B_NK ? ptx::smem_desc_sw128(b_src + k * (UMMA_K * 2), 16, 1024)
                                          : ptx::smem_desc_sw128(b_src + k * (UMMA_K * 128), B_ATOM_BYTES, 1024);
              ptx::mma_bf16(tmem_base + a * UMMA_N, adesc, bdesc, idesc, (kb | static_cast<uint32_t>(k)) != 0u);
            }
          }
          if (!ok) break;
          ptx::mma_commit(ptx::smem_u32(&bar_empty[stage]));  // the stage is free once these MMAs have read it
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (ok) ptx::mma_commit(ptx::smem_u32(&bar_tmem_full));  // both accumulators complete
      }
    }
  } else {
    // ---------------- epilogue ----------------
    const int e = warp - 2;
    const uint32_t quad = static_cast<uint32_t>(warp) & 3u;  // TMEM lanes a warp may read: 32 * (warp % 4)
    const uint32_t half = static_cast<uint32_t>(e) >> 2;     // which 128 of the 256 columns
    const uint32_t stage_box = smem_base + STAGES * STAGE_BYTES + e * EPI_BOX_BYTES;  // 1024-byte aligned
    uint32_t tile_iter = 0;
    bool ok = true;
    // No early exit from this loop: the named barriers below need every epilogue warp, every tile. A
    // warp that gave up on a wait keeps walking the tiles and only skips the work.
    for (uint32_t t = blockIdx.x; t < num_tiles; t += gridDim.x, ++tile_iter) {
      const TileCoord tc = tile_coord(t, tiles_m, tiles_n);
      // The tile's 256 bias values go to shared memory while the K loop runs; a global load inside the
      // drain would sit on the critical path.
      ptx::named_bar_sync(1, EPI_WARPS * 32);  // every warp has finished reading the previous tile's values
      {
        const uint32_t et = threadIdx.x - 64u, col = tc.n * BN + et;
        bias_s[et] = (bias != nullptr && col < N) ? __ldg(bias + col) : 0.0f;
      }
      ptx::named_bar_sync(1, EPI_WARPS * 32);
      if (ok && num_kb > 0) {
        if (!ptx::mbar_wait(ptx::smem_u32(&bar_tmem_full), tile_iter & 1u, abort_p)) ok = false;
        ptx::tc_fence_after();
      }
      if (!ok) continue;
      // Eight half boxes of 32 columns per warp and tile, four per accumulator. What the next tile's K loop
      // waits for is the accumulator, not the stores: a warp first pulls its whole share of accumulator 0
      // into registers (128 values per thread) and hands the accumulator back, then converts and stores from
      // registers; each register block that has been staged is refilled from accumulator 1 at once, so that
      // accumulator 1 is handed back as soon as the last of accumulator 0's half boxes is staged.
      const uint32_t tm_warp = tmem_base + ((quad * 32u) << 16) + half * 128;
      uint32_t r[4][32];
      if (num_kb > 0) {
#pragma unroll
        for (uint32_t q = 0; q < 4; ++q) ptx::tmem_ld_32x32(tm_warp + q * 32, r[q]);
#pragma unroll
        for (uint32_t q = 0; q < 4; ++q) ptx::tmem_ld_wait_for(r[q]);
        ptx::tc_fence_before();
        if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&bar_tmem_empty[0]));
      } else {
#pragma unroll
        for (uint32_t q = 0; q < 4; ++q)
#pragma unroll
          for (int j = 0; j < 32; ++j) r[q][j] = 0u;  // empty reduction: the accumulator's init
      }
#pragma unroll
      for (uint32_t i = 0; i < 8; ++i) {
        const uint32_t a = i >> 2, q = i & 3u, cbase = q * 32;  // accumulator, register block, first column
        const uint32_t row0 = tc.m * BM + a * UMMA_M + quad * 32;
        const uint32_t col0 = tc.n * BN + half * 128 + cbase;
        const uint32_t buf = OUT_F32 ? stage_box : stage_box + (i & 1u) * (EPI_BOX_BYTES / 2);
        if (i == 4 && num_kb > 0) {  // accumulator 1 is in registers
#pragma unroll
          for (uint32_t qq = 0; qq < 4; ++qq) ptx::tmem_ld_wait_for(r[qq]);
          ptx::tc_fence_before();
          if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&bar_tmem_empty[1]));
        }
        // two staging buffers alternate: the store issued two half boxes ago has left this one (an fp32 half box
        // fills the warp's whole staging space: the previous store must have left it)
        if (lane == 0) {
          if (OUT_F32) ptx::tma_store_wait_read();
          else ptx::tma_store_wait_read_1();
        }
        __syncwarp();
        if (OUT_F32) stage_half_box_f32(r[q], alpha, buf, lane);
        else stage_half_box(r[q], bias_s + half * 128 + cbase, act, buf, lane);
        if (i < 4 && num_kb > 0) ptx::tmem_ld_32x32(tm_warp + UMMA_N + q * 32, r[q]);  // refill from accumulator 1
        ptx::fence_proxy_async();  // the TMA engine reads what the threads just wrote
        __syncwarp();
        if (lane == 0) {
          // a box that starts inside the tensor; the hardware clips its edges. A box that lies outside still commits
          // an (empty) group: the wait above counts groups, and with a group missing it would let this warp restage
          // a buffer whose store is still being read (N = 256 j + 129 ... 160: a stored box, then three skipped ones)
          if (row0 < M && col0 < N) ptx::tma_store_2d(&tmap_c, buf, static_cast<int32_t>(col0), static_cast<int32_t>(row0));
          ptx::tma_store_commit();
        }
      }
    }
    if (lane == 0) ptx::tma_store_wait_all();  // every box has reached global memory before the CTA exits
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, TMEM_COLS);
  }
  if (threadIdx.x == 0 && abort_flag != 0) g_gemm_status = 1;
}

// ---------------------------------------------------------------------------------------------
// The same contraction on CTA PAIRS (cta_group::2): a cluster of two CTAs owns a 512x256 output
// tile. Each tcgen05.mma has M = 256 -- 128 rows in each CTA's TMEM -- and N = 256; every CTA loads
// only ITS rows of A and ITS half of B's columns (the tensor cores read the other half from the
// peer's shared memory), so a K block costs a CTA 48 KB instead of 64 KB for the same 8.4 MFLOP and
// the ring holds four stages instead of three. Only the leader CTA (cluster rank 0) issues MMAs; its
// commits arrive on the barriers of both CTAs. No load has more than one destination.
// ---------------------------------------------------------------------------------------------
constexpr int P_STAGES = 4;
constexpr int P_A_STAGE_BYTES = 2 * UMMA_M * 128;   // this CTA's 128 rows of both accumulators: 32 KB
constexpr int P_B_STAGE_BYTES = BK * (BN / 2) * 2;  // this CTA's 128 columns of B: 16 KB (2 boxes)
constexpr int P_STAGE_BYTES = P_A_STAGE_BYTES + P_B_STAGE_BYTES;
constexpr int P_BM = 512;
constexpr size_t P_SMEM_BYTES = static_cast<size_t>(P_STAGES) * P_STAGE_BYTES + EPI_WARPS * EPI_BOX_BYTES + 1024;

__global__ void __launch_bounds__(THREADS, 1)
gemm_bias_act_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                          const __grid_constant__ CUtensorMap tmap_c, const float* __restrict__ bias, uint32_t M,
                          uint32_t N, uint32_t K, int act) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_full[P_STAGES];    // used in the leader: bytes of BOTH CTAs land here
  __shared__ __align__(8) uint64_t bar_empty[P_STAGES];   // in each CTA: the leader's commit arrives on both
  __shared__ __align__(8) uint64_t bar_tmem_full;         // in each CTA
  __shared__ __align__(8) uint64_t bar_tmem_empty[2];     // used in the leader: epilogue warps of both CTAs arrive
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = ptx::cluster_ctarank();
  const bool leader = rank == 0;
  volatile int* abort_p = &abort_flag;

  const uint32_t tiles_m = (M + P_BM - 1) / P_BM, tiles_n = (N + BN - 1) / BN;
  const uint32_t num_tiles = tiles_m * tiles_n;
  const uint32_t num_kb = (K + BK - 1) / BK;
  const uint32_t pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < P_STAGES; ++s) {
      ptx::mbar_init(ptx::smem_u32(&bar_full[s]), 1);
      ptx::mbar_init(ptx::smem_u32(&bar_empty[s]), 1);
    }
    ptx::mbar_init(ptx::smem_u32(&bar_tmem_full), 1);
    ptx::mbar_init(ptx::smem_u32(&bar_tmem_empty[0]), 2 * EPI_WARPS);
    ptx::mbar_init(ptx::smem_u32(&bar_tmem_empty[1]), 2 * EPI_WARPS);
    ptx::fence_barrier_init();
    ptx::fence_proxy_async();
    ptx::prefetch_tensormap(&tmap_a);
    ptx::prefetch_tensormap(&tmap_b);
    ptx::prefetch_tensormap(&tmap_c);
  }
  if (warp == 1) {
    ptx::tmem_alloc_pair(ptx::smem_u32(&tmem_base_slot), TMEM_COLS);
    ptx::tmem_relinquish_pair();
  }
  ptx::tc_fence_before();
  __syncthreads();
  // the peer's barriers must be initialised before anything of this CTA can signal them
  ptx::cluster_arrive();
  ptx::cluster_wait();
  ptx::tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;

  if (warp == 0) {
    // ---------------- TMA producer (both CTAs) ----------------
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (uint32_t t = pair; ok && t < num_tiles; t += num_pairs) {
        const TileCoord tc = tile_coord(t, tiles_m, tiles_n);
        for (uint32_t kb = 0; kb < num_kb; ++kb) {
          if (!ptx::mbar_wait(ptx::smem_u32(&bar_empty[stage]), phase ^ 1u, abort_p)) { ok = false; break; }
          const uint32_t full_leader = ptx::mapa(ptx::smem_u32(&bar_full[stage]), 0);
          const uint32_t a_dst = smem_base + stage * P_STAGE_BYTES;
          const uint32_t b_dst = a_dst + P_A_STAGE_BYTES;
          if (leader) ptx::mbar_expect_tx(ptx::smem_u32(&bar_full[stage]), 2 * P_STAGE_BYTES);
#pragma unroll
          for (int a = 0; a < 2; ++a)  // accumulator a covers rows [a*256, a*256+256) of the tile; mine: + rank*128
            ptx::tma_load_2d_pair(a_dst + a * (UMMA_M * 128), &tmap_a, full_leader, static_cast<int32_t>(kb * BK),
                                  static_cast<int32_t>(tc.m * P_BM + a * 256 + rank * UMMA_M));
#pragma unroll
          for (int j = 0; j < 2; ++j)  // my 128 columns of B
            ptx::tma_load_2d_pair(b_dst + j * B_ATOM_BYTES, &tmap_b, full_leader,
                                  static_cast<int32_t>(tc.n * BN + rank * 128 + j * 64), static_cast<int32_t>(kb * BK));
          if (++stage == P_STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (leader CTA only) ----------------
    if (leader && lane == 0) {
      constexpr uint32_t idesc = ptx::idesc_bf16_f32(2 * UMMA_M, UMMA_N, /*a_mn=*/0, /*b_mn=*/1);
      uint32_t stage = 0, phase = 0, tile_iter = 0;
      bool ok = true;
      for (uint32_t t = pair; ok && t < num_tiles; t += num_pairs, ++tile_iter) {
        for (uint32_t kb = 0; ok && kb < num_kb; ++kb) {
          if (!ptx::mbar_wait(ptx::smem_u32(&bar_full[stage]), phase, abort_p)) { ok = false; break; }
          ptx::tc_fence_after();
          const uint32_t a_src = smem_base + stage * P_STAGE_BYTES;
          const uint32_t b_src = a_src + P_A_STAGE_BYTES;
#pragma unroll
          for (int a = 0; a < 2; ++a) {
            if (kb == 0) {
              if (!ptx::mbar_wait(ptx::smem_u32(&bar_tmem_empty[a]), (tile_iter & 1u) ^ 1u, abort_p)) { ok = false; break; }
              ptx::tc_fence_after();
            }
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k) {
              const uint64_t adesc = ptx::smem_desc_sw128(a_src + a * (UMMA_M * 128) + k * (UMMA_K * 2), 16, 1024);
              const uint64_t bdesc = ptx::smem_desc_sw128(b_src + k * (UMMA_K * 128), B_ATOM_BYTES, 1024);
              ptx::mma_bf16_pair(tmem_base + a * UMMA_N, adesc, bdesc, idesc, (kb | static_cast<uint32_t>(k)) != 0u);
            }
          }
          if (!ok) break;
          ptx::mma_commit_pair(ptx::smem_u32(&bar_empty[stage]), 3);  // frees the stage in both CTAs
          if (++stage == P_STAGES) { stage = 0; phase ^= 1u; }
        }
        if (ok) ptx::mma_commit_pair(ptx::smem_u32(&bar_tmem_full), 3);  // wakes the epilogues of both CTAs
      }
    }
  } else {
    // ---------------- epilogue (both CTAs, each drains its own 128 rows) ----------------
    const int e = warp - 2;
    const uint32_t quad = static_cast<uint32_t>(warp) & 3u;
    const uint32_t half = static_cast<uint32_t>(e) >> 2;
    const uint32_t stage_box = smem_base + P_STAGES * P_STAGE_BYTES + e * EPI_BOX_BYTES;
    const uint32_t my_row = stage_box + lane * 128;
    const bool bias_vec = bias != nullptr && (reinterpret_cast<uintptr_t>(bias) & 15u) == 0;
    uint32_t tile_iter = 0;
    bool ok = true;
    for (uint32_t t = pair; ok && t < num_tiles; t += num_pairs, ++tile_iter) {
      const TileCoord tc = tile_coord(t, tiles_m, tiles_n);
      const BiasRegs breg = load_bias_regs(bias, bias_vec, tc.n * BN + half * 128 + lane * 4, N);
      if (num_kb > 0) {
        if (!ptx::mbar_wait(ptx::smem_u32(&bar_tmem_full), tile_iter & 1u, abort_p)) { ok = false; break; }
        ptx::tc_fence_after();
      }
#pragma unroll 1
      for (uint32_t a = 0; a < 2; ++a) {
        const uint32_t row0 = tc.m * P_BM + a * 256 + rank * UMMA_M + quad * 32;
#pragma unroll 1
        for (uint32_t grp = 0; grp < 2; ++grp) {
          const uint32_t col0 = tc.n * BN + half * 128 + grp * 64;
          if (lane == 0) ptx::tma_store_wait_read();
          __syncwarp();
          stage_box_from_tmem(tmem_base + ((quad * 32u) << 16) + a * UMMA_N + half * 128 + grp * 64, num_kb > 0, breg,
                              grp * 64, act, my_row, lane);
          if (grp == 1) ptx::tc_fence_before();
          ptx::fence_proxy_async();
          __syncwarp();
          if (lane == 0) {
            // hand the accumulator back: the leader's barrier counts the epilogue warps of both CTAs
            if (grp == 1) ptx::mbar_arrive_cluster(ptx::mapa(ptx::smem_u32(&bar_tmem_empty[a]), 0));
            if (row0 < M && col0 < N) {
              ptx::tma_store_2d(&tmap_c, stage_box, static_cast<int32_t>(col0), static_cast<int32_t>(row0));
              ptx::tma_store_commit();
            }
          }
        }
      }
    }
    if (lane == 0) ptx::tma_store_wait_all();
  }

  ptx::tc_fence_before();
  __syncthreads();
  // neither CTA may exit (or free TMEM) while the other can still signal its barriers or read its
  // shared memory through the tensor core
  ptx::cluster_arrive();
  ptx::cluster_wait();
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
  if (threadIdx.x == 0 && abort_flag != 0) g_gemm_status = 2;
}

// ---------------------------------------------------------------------------------------------
// Double-buffered accumulators. The two kernels above give a tile all 512 TMEM columns, so the
// tensor pipe idles while the epilogue drains a tile. Here a CTA's share of a tile is 128 rows x
// 256 columns = 256 TMEM columns, two such accumulators alternate by tile parity, and the
// epilogue of tile i runs under the K loop of tile i+1.
//   PAIR = false: one CTA per 128x256 tile; a K block costs 48 KB (A 128x64 + B 64x256), 4 stages.
//   PAIR = true : a cluster of two CTAs per 256x256 tile with cta_group::2 (M = 256): each CTA
//                 loads its 128 rows of A and its 128 columns of B, 32 KB per K block, 6 stages;
//                 the leader issues the MMAs and its commits arrive on both CTAs' barriers.
// ---------------------------------------------------------------------------------------------
template <bool PAIR>
struct Db {
  static constexpr int CTAS = PAIR ? 2 : 1;
  static constexpr int TILE_M = UMMA_M * CTAS;
  static constexpr int B_COLS = BN / CTAS;
  static constexpr int A_BYTES = UMMA_M * 128;           // 16 KB
  static constexpr int B_BYTES = BK * B_COLS * 2;        // 32 KB / 16 KB
  static constexpr int STAGE = A_BYTES + B_BYTES;
  static constexpr int STAGES = PAIR ? 6 : 4;
  static constexpr size_t SMEM = static_cast<size_t>(STAGES) * STAGE + EPI_WARPS * EPI_BOX_BYTES + 1024;
};

template <bool PAIR>
__global__ void __launch_bounds__(THREADS, 1)
gemm_bias_act_db_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                        const __grid_constant__ CUtensorMap tmap_c, const float* __restrict__ bias, uint32_t M,
                        uint32_t N, uint32_t K, int act, uint32_t ksplit, uint32_t kb_per_split,
                        float* __restrict__ partial, uint32_t* __restrict__ counters, __nv_bfloat16* __restrict__ c_raw) {
  // ksplit > 1: a unit of work is (tile, range of K blocks); its fp32 accumulator goes to
  // partial[range][M][N] as it is. With `counters` (one per tile, CTA of the pair and epilogue warp, all zero
  // between launches) the epilogue warp that arrives LAST at its 32 x 128 block of the tile adds the ranges in
  // ascending order, the bias and the activation and stores c; every other warp only publishes its partial.
  // Nobody waits for anybody: the last arriver is whoever finds the counter at ksplit - 1. Without `counters`
  // gemm_split_finish does the adding in a second launch.
  using C = Db<PAIR>;
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_full[C::STAGES];   // PAIR: used in the leader, bytes of both CTAs land here
  __shared__ __align__(8) uint64_t bar_empty[C::STAGES];  // in each CTA
  __shared__ __align__(8) uint64_t bar_tmem_full[2];      // in each CTA, one per accumulator
  __shared__ __align__(8) uint64_t bar_tmem_empty[2];     // PAIR: used in the leader, all epilogue warps arrive
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = PAIR ? ptx::cluster_ctarank() : 0u;
  const bool leader = rank == 0;
  volatile int* abort_p = &abort_flag;

  const uint32_t tiles_m = (M + C::TILE_M - 1) / C::TILE_M, tiles_n = (N + BN - 1) / BN;
  const uint32_t num_tiles = tiles_m * tiles_n * ksplit;  // units of work
  const uint32_t all_kb = (K + BK - 1) / BK;
  const uint32_t first = PAIR ? blockIdx.x >> 1 : blockIdx.x, step = PAIR ? gridDim.x >> 1 : gridDim.x;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < C::STAGES; ++s) {
      ptx::mbar_init(ptx::smem_u32(&bar_full[s]), 1);
      ptx::mbar_init(ptx::smem_u32(&bar_empty[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      ptx::mbar_init(ptx::smem_u32(&bar_tmem_full[a]), 1);
      ptx::mbar_init(ptx::smem_u32(&bar_tmem_empty[a]), C::CTAS * EPI_WARPS);
    }
    ptx::fence_barrier_init();
    ptx::fence_proxy_async();
    ptx::prefetch_tensormap(&tmap_a);
    ptx::prefetch_tensormap(&tmap_b);
    ptx::prefetch_tensormap(&tmap_c);
  }
  if (warp == 1) {
    if (PAIR) {
      ptx::tmem_alloc_pair(ptx::smem_u32(&tmem_base_slot), TMEM_COLS);
      ptx::tmem_relinquish_pair();
    } else {
      ptx::tmem_alloc(ptx::smem_u32(&tmem_base_slot), TMEM_COLS);
      ptx::tmem_relinquish();
    }
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (PAIR) {  // the peer's barriers must be initialised before anything of this CTA can signal them
    ptx::cluster_arrive();
    ptx::cluster_wait();
  }
  ptx::tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;

  if (warp == 0) {
    // ---------------- TMA producer (every CTA) ----------------
    // Lane 0 loads A, lanes 1.. load one 64-column box of B each: the boxes of a stage go out with one
    // warp instruction instead of one instruction after the other from a single thread.
    constexpr int B_BOXES = C::B_COLS / 64;
    uint32_t stage = 0, phase = 0;
    bool ok = true;
    for (uint32_t t = first; ok && t < num_tiles; t += step) {
      const TileCoord tc = tile_coord(t / ksplit, tiles_m, tiles_n);
      const uint32_t kb0 = (t % ksplit) * kb_per_split;
      const uint32_t num_kb = kb0 < all_kb ? (all_kb - kb0 < kb_per_split ? all_kb - kb0 : kb_per_split) : 0u;
      const int32_t a_row = static_cast<int32_t>(tc.m * C::TILE_M + rank * UMMA_M);
      const int32_t b_col = static_cast<int32_t>(tc.n * BN + rank * C::B_COLS);
      for (uint32_t kb = 0; kb < num_kb; ++kb) {
        if (!ptx::mbar_wait(ptx::smem_u32(&bar_empty[stage]), phase ^ 1u, abort_p)) { ok = false; break; }
        const uint32_t a_dst = smem_base + stage * C::STAGE;
        const uint32_t b_dst = a_dst + C::A_BYTES;
        const int32_t k0 = static_cast<int32_t>((kb0 + kb) * BK);
        const uint32_t full = PAIR ? ptx::mapa(ptx::smem_u32(&bar_full[stage]), 0) : ptx::smem_u32(&bar_full[stage]);
        if (lane == 0) {
          if (leader) ptx::mbar_expect_tx(ptx::smem_u32(&bar_full[stage]), C::CTAS * C::STAGE);
          if (PAIR) ptx::tma_load_2d_pair(a_dst, &tmap_a, full, k0, a_row);
          else ptx::tma_load_2d(a_dst, &tmap_a, full, k0, a_row);
        } else if (lane <= B_BOXES) {
          const int j = lane - 1;
          if (PAIR) ptx::tma_load_2d_pair(b_dst + j * B_ATOM_BYTES, &tmap_b, full, b_col + j * 64, k0);
          else ptx::tma_load_2d(b_dst + j * B_ATOM_BYTES, &tmap_b, full, b_col + j * 64, k0);
        }
        if (++stage == C::STAGES) { stage = 0; phase ^= 1u; }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (the leader CTA) ----------------
    if (leader && lane == 0) {
      constexpr uint32_t idesc = ptx::idesc_bf16_f32(C::TILE_M, UMMA_N, /*a_mn=*/0, /*b_mn=*/1);
      uint32_t stage = 0, phase = 0, tile_iter = 0;
      bool ok = true;
      for (uint32_t t = first; ok && t < num_tiles; t += step, ++tile_iter) {
        const uint32_t acc = tile_iter & 1u, use = (tile_iter >> 1) & 1u;
        const uint32_t kb0 = (t % ksplit) * kb_per_split;
        const uint32_t num_kb = kb0 < all_kb ? (all_kb - kb0 < kb_per_split ? all_kb - kb0 : kb_per_split) : 0u;
        if (num_kb > 0) {  // the epilogue must have drained this accumulator (two tiles ago)
          if (!ptx::mbar_wait(ptx::smem_u32(&bar_tmem_empty[acc]), use ^ 1u, abort_p)) break;
          ptx::tc_fence_after();
        }
        for (uint32_t kb = 0; kb < num_kb; ++kb) {
          if (!ptx::mbar_wait(ptx::smem_u32(&bar_full[stage]), phase, abort_p)) { ok = false; break; }
          ptx::tc_fence_after();
          const uint32_t a_src = smem_base + stage * C::STAGE;
          const uint32_t b_src = a_src + C::A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t adesc = ptx::smem_desc_sw128(a_src + k * (UMMA_K * 2), 16, 1024);
            const uint64_t bdesc = ptx::smem_desc_sw128(b_src + k * (UMMA_K * 128), B_ATOM_BYTES, 1024);
            if (PAIR) ptx::mma_bf16_pair(tmem_base + acc * UMMA_N, adesc, bdesc, idesc, (kb | static_cast<uint32_t>(k)) != 0u);
            else ptx::mma_bf16(tmem_base + acc * UMMA_N, adesc, bdesc, idesc, (kb | static_cast<uint32_t>(k)) != 0u);
          }
          if (PAIR) ptx::mma_commit_pair(ptx::smem_u32(&bar_empty[stage]), 3);
          else ptx::mma_commit(ptx::smem_u32(&bar_empty[stage]));
          if (++stage == C::STAGES) { stage = 0; phase ^= 1u; }
        }
        if (ok && num_kb > 0) {
          if (PAIR) ptx::mma_commit_pair(ptx::smem_u32(&bar_tmem_full[acc]), 3);
          else ptx::mma_commit(ptx::smem_u32(&bar_tmem_full[acc]));
        }
      }
    }
  } else {
    // ---------------- epilogue (every CTA drains its own 128 rows) ----------------
    const int e = warp - 2;
    const uint32_t quad = static_cast<uint32_t>(warp) & 3u;
    const uint32_t half = static_cast<uint32_t>(e) >> 2;
    const uint32_t stage_box = smem_base + C::STAGES * C::STAGE + e * EPI_BOX_BYTES;
    const uint32_t my_row = stage_box + lane * 128;
    const bool bias_vec = bias != nullptr && (reinterpret_cast<uintptr_t>(bias) & 15u) == 0;
    uint32_t tile_iter = 0;
    bool ok = true;
    for (uint32_t t = first; ok && t < num_tiles; t += step, ++tile_iter) {
      const TileCoord tc = tile_coord(t / ksplit, tiles_m, tiles_n);
      const uint32_t ks = t % ksplit, kb0 = ks * kb_per_split;
      const uint32_t num_kb = kb0 < all_kb ? (all_kb - kb0 < kb_per_split ? all_kb - kb0 : kb_per_split) : 0u;
      const uint32_t acc = tile_iter & 1u, use = (tile_iter >> 1) & 1u;
      const BiasRegs breg = load_bias_regs(bias, bias_vec, tc.n * BN + half * 128 + lane * 4, N);
      if (num_kb > 0) {
        if (!ptx::mbar_wait(ptx::smem_u32(&bar_tmem_full[acc]), use, abort_p)) { ok = false; break; }
        ptx::tc_fence_after();
      }
      const uint32_t row0 = tc.m * C::TILE_M + rank * UMMA_M + quad * 32;
      if (ksplit > 1) {
        // fp32 partial of this K range, straight from TMEM: a thread owns a row and writes 32 consecutive columns
        // (one 128-byte line) per load
        const uint32_t row = row0 + lane;
        float* prow = partial + (static_cast<size_t>(ks) * M + row) * N;
#pragma unroll 1
        for (uint32_t q = 0; q < 4; ++q) {
          const uint32_t col = tc.n * BN + half * 128 + q * 32;
          uint32_t r[32];
          if (num_kb > 0) {
            ptx::tmem_ld_32x32(tmem_base + ((quad * 32u) << 16) + acc * UMMA_N + half * 128 + q * 32, r);
            ptx::tmem_ld_wait_for(r);
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) r[j] = 0u;
          }
          if (row < M) {
#pragma unroll
            for (int v = 0; v < 8; ++v)
              if (col + v * 4 < N)  // N % 8 == 0: groups of four columns are inside or outside as a whole
                *reinterpret_cast<uint4*>(prow + col + v * 4) = make_uint4(r[v * 4], r[v * 4 + 1], r[v * 4 + 2], r[v * 4 + 3]);
          }
        }
        if (num_kb > 0) {
          ptx::tc_fence_before();
          __syncwarp();
          if (lane == 0) {
            if (PAIR) ptx::mbar_arrive_cluster(ptx::mapa(ptx::smem_u32(&bar_tmem_empty[acc]), 0));
            else ptx::mbar_arrive(ptx::smem_u32(&bar_tmem_empty[acc]));
          }
        }
        if (counters != nullptr) {
          __threadfence();  // this lane's partial stores are visible device-wide before the count below
          __syncwarp();
          uint32_t* ctr = counters + ((t / ksplit) * C::CTAS + rank) * EPI_WARPS + e;
          uint32_t last = 0;
          if (lane == 0) {
            last = atomicAdd(ctr, 1u) == ksplit - 1 ? 1u : 0u;
            if (last) *ctr = 0u;  // every range of this block has arrived: ready for the next launch
          }
          last = __shfl_sync(0xffffffffu, last, 0);
          if (last) {
            __threadfence();  // the other ranges' partials, published before their counts, are visible now
            // the warp's 32 x 128 block, four rows at a time: a lane owns four columns, so a row of a range is one
            // coalesced 512-byte load and the loads of all ranges and rows of a step are in flight together
            const uint32_t colbase = tc.n * BN + half * 128 + lane * 4;
            const bool col_ok = colbase < N;  // N % 8 == 0: groups of four columns are inside or outside as a whole
            float4 bv = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (bias != nullptr && col_ok) bv = make_float4(__ldg(bias + colbase), __ldg(bias + colbase + 1), __ldg(bias + colbase + 2), __ldg(bias + colbase + 3));
#pragma unroll 1
            for (uint32_t r0 = 0; r0 < 32; r0 += 4) {
              float4 sum[4];
#pragma unroll
              for (int i = 0; i < 4; ++i) sum[i] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll 4
              for (uint32_t r2 = 0; r2 < ksplit; ++r2) {  // ascending ranges: ascending k, like the one-pass kernel
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  const uint32_t ri = row0 + r0 + i;
                  if (ri < M && col_ok) {  // read around L1: these lines were written by other SMs
                    const float4 pv = __ldcg(reinterpret_cast<const float4*>(partial + (static_cast<size_t>(r2) * M + ri) * N + colbase));
                    sum[i].x += pv.x; sum[i].y += pv.y; sum[i].z += pv.z; sum[i].w += pv.w;
                  }
                }
              }
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const uint32_t ri = row0 + r0 + i;
                if (ri >= M || !col_ok) continue;
                float f0 = sum[i].x + bv.x, f1 = sum[i].y + bv.y, f2 = sum[i].z + bv.z, f3 = sum[i].w + bv.w;
                if (act == TCAB_ACT_RELU) {
                  f0 = fmaxf(f0, 0.0f); f1 = fmaxf(f1, 0.0f); f2 = fmaxf(f2, 0.0f); f3 = fmaxf(f3, 0.0f);
                }
                const __nv_bfloat162 h0 = __floats2bfloat162_rn(f0, f1), h1 = __floats2bfloat162_rn(f2, f3);
                *reinterpret_cast<uint2*>(c_raw + static_cast<size_t>(ri) * N + colbase) =
                    make_uint2(*reinterpret_cast<const uint32_t*>(&h0), *reinterpret_cast<const uint32_t*>(&h1));
              }
            }
          }
        }
        continue;
      }
#pragma unroll 1
      for (uint32_t grp = 0; grp < 2; ++grp) {
        const uint32_t col0 = tc.n * BN + half * 128 + grp * 64;
        if (lane == 0) ptx::tma_store_wait_read();  // the previous box has left shared memory
        __syncwarp();
        stage_box_from_tmem(tmem_base + ((quad * 32u) << 16) + acc * UMMA_N + half * 128 + grp * 64, num_kb > 0, breg,
                            grp * 64, act, my_row, lane);
        if (grp == 1) ptx::tc_fence_before();
        ptx::fence_proxy_async();
        __syncwarp();
        if (lane == 0) {
          if (grp == 1 && num_kb > 0) {  // hand the accumulator back to the MMA issuer
            if (PAIR) ptx::mbar_arrive_cluster(ptx::mapa(ptx::smem_u32(&bar_tmem_empty[acc]), 0));
            else ptx::mbar_arrive(ptx::smem_u32(&bar_tmem_empty[acc]));
          }
          if (row0 < M && col0 < N) {
            ptx::tma_store_2d(&tmap_c, stage_box, static_cast<int32_t>(col0), static_cast<int32_t>(row0));
            ptx::tma_store_commit();
          }
        }
      }
    }
    if (lane == 0) ptx::tma_store_wait_all();
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (PAIR) {  // neither CTA may exit or free TMEM while the other can still signal it or read its shared memory
    ptx::cluster_arrive();
    ptx::cluster_wait();
  }
  if (warp == 1) {
    ptx::tc_fence_after();
    if (PAIR) ptx::tmem_dealloc_pair(tmem_base, TMEM_COLS);
    else ptx::tmem_dealloc(tmem_base, TMEM_COLS);
  }
  if (threadIdx.x == 0 && abort_flag != 0) g_gemm_status = PAIR ? 4 : 3;
}

// ------------------------------------------------------------------------------------------------------------
// Few output tiles and a long K: the K ranges of one 128 x 256 tile run on the CTAs of ONE thread-block cluster
// (KS = 2..8 CTAs, one unit of work each). Every CTA accumulates its range in TMEM and copies the fp32 accumulator
// into its own shared memory (over the drained operand ring). The tile's rows are dealt out to the CTAs of the
// cluster: a CTA writes the rows it does not own to a workspace (they stay in L2), the cluster synchronises, and
// each CTA adds, for its own rows, the ranges in ascending order -- its own from shared memory, the others' from
// the workspace -- then the bias and the activation, and stores bf16. One launch; every SM of the cluster takes an
// equal share of the adding. (Reading the peers' accumulators through distributed shared memory instead was
// measured at 8 us for a 128 x 256 tile in four ranges: the SM-to-SM path is slower than L2.) The sum is taken in
// the same order as gemm_split_finish takes it: the forms give the same bits.
// ------------------------------------------------------------------------------------------------------------
struct Ck {
  static constexpr int A_BYTES = UMMA_M * 128;            // 16 KB: 128 rows x 64 bf16
  static constexpr int B_BYTES = BK * BN * 2;             // 32 KB
  static constexpr int STAGE = A_BYTES + B_BYTES;
  static constexpr int STAGES = 4;
  static constexpr int PLANE_BYTES = UMMA_M * BN * 4;     // the fp32 accumulator: 128 rows x 1 KB
  static constexpr size_t SMEM = static_cast<size_t>(STAGES) * STAGE + 1024;
  static_assert(PLANE_BYTES <= STAGES * STAGE, "the accumulator plane lies over the operand ring");
};

__device__ __forceinline__ float4 ld_shared_v4(uint32_t addr) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr) : "memory");
  return v;
}

// OUT_F32: c is fp32 (c_f32, rows c_pitch elements apart) and receives alpha * sum, no bias, no activation: the
// product chains of tcab_chain_contract; B_NK: b is [N, K] (one K-major box of 256 rows per stage).
template <int KS, bool OUT_F32 = false, bool B_NK = false>
__global__ void __launch_bounds__(THREADS, 1)
gemm_cluster_k_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                      const float* __restrict__ bias, uint32_t M, uint32_t N, uint32_t K, int act,
                      uint32_t kb_per_split, float* __restrict__ ws, __nv_bfloat16* __restrict__ c_raw,
                      float* __restrict__ c_f32, uint64_t c_pitch, float alpha) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_full[Ck::STAGES];
  __shared__ __align__(8) uint64_t bar_empty[Ck::STAGES];
  __shared__ __align__(8) uint64_t bar_tmem_full;
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = ptx::cluster_ctarank();  // the K range; clusters are KS x 1 x 1 over a 1-D grid
  volatile int* abort_p = &abort_flag;

  const uint32_t tiles_m = (M + UMMA_M - 1) / UMMA_M, tiles_n = (N + BN - 1) / BN;
  const uint32_t tile = blockIdx.x / KS;
  const TileCoord tc = tile_coord(tile, tiles_m, tiles_n);
  const uint32_t all_kb = (K + BK - 1) / BK;
  const uint32_t kb0 = rank * kb_per_split;
  const uint32_t num_kb = kb0 < all_kb ? (all_kb - kb0 < kb_per_split ? all_kb - kb0 : kb_per_split) : 0u;
  constexpr uint32_t ROWS_PER = (UMMA_M + KS - 1) / KS;  // rows of the tile a CTA adds and stores
  const uint32_t rows_here = min(static_cast<uint32_t>(UMMA_M), M - tc.m * UMMA_M);  // rows of the tile inside c

  // Warp 0 initialises the barriers and has the first copies under way before the rest of the CTA is set up
  // (the TMEM allocation, the CTA-wide barrier): the first bytes from HBM are what the kernel waits for longest.
  const int32_t a_row = static_cast<int32_t>(tc.m * UMMA_M), b_col = static_cast<int32_t>(tc.n * BN);
  auto load_stage = [&](uint32_t kb, uint32_t stage) {
    const uint32_t a_dst = smem_base + stage * Ck::STAGE, b_dst = a_dst + Ck::A_BYTES;
    const int32_t k0 = static_cast<int32_t>((kb0 + kb) * BK);
    const uint32_t full = ptx::smem_u32(&bar_full[stage]);
    if (lane == 0) {
      ptx::mbar_expect_tx(full, Ck::STAGE);
      ptx::tma_load_2d(a_dst, &tmap_a, full, k0, a_row);
      if (B_NK) ptx::tma_load_2d(b_dst, &tmap_b, full, k0, b_col);  // one box: 256 rows of n, 64 of k
    } else if (!B_NK && lane <= BN / 64) {
      const int j = lane - 1;
      ptx::tma_load_2d(b_dst + j * B_ATOM_BYTES, &tmap_b, full, b_col + j * 64, k0);
    }
  };
  const uint32_t early = num_kb < static_cast<uint32_t>(Ck::STAGES) ? num_kb : static_cast<uint32_t>(Ck::STAGES);
  if (warp == 0) {
    if (lane == 0) {
      ptx::prefetch_tensormap(&tmap_a);
      ptx::prefetch_tensormap(&tmap_b);
      abort_flag = 0;
      for (int s = 0; s < Ck::STAGES; ++s) {
        ptx::mbar_init(ptx::smem_u32(&bar_full[s]), 1);
        ptx::mbar_init(ptx::smem_u32(&bar_empty[s]), 1);
      }
      ptx::mbar_init(ptx::smem_u32(&bar_tmem_full), 1);
      ptx::fence_barrier_init();
      ptx::fence_proxy_async();
    }
    __syncwarp();
    for (uint32_t kb = 0; kb < early; ++kb) load_stage(kb, kb);  // the ring is empty: nothing to wait for
  }
  if (warp == 1) {
    ptx::tmem_alloc(ptx::smem_u32(&tmem_base_slot), UMMA_N);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;

  float bv[2][4];  // epilogue warps: the bias of the lane's two groups of four columns
  if (warp == 0) {
    // ---------------- TMA producer: lane 0 loads A, lanes 1..4 one 64-column box of B each ----------------
    uint32_t stage = early == static_cast<uint32_t>(Ck::STAGES) ? 0u : early, phase = early == static_cast<uint32_t>(Ck::STAGES) ? 1u : 0u;
    for (uint32_t kb = early; kb < num_kb; ++kb) {
      if (!ptx::mbar_wait(ptx::smem_u32(&bar_empty[stage]), phase ^ 1u, abort_p)) break;
      load_stage(kb, stage);
      if (++stage == Ck::STAGES) { stage = 0; phase ^= 1u; }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t idesc = ptx::idesc_bf16_f32(UMMA_M, UMMA_N, /*a_mn=*/0, /*b_mn=*/B_NK ? 0 : 1);
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (uint32_t kb = 0; kb < num_kb; ++kb) {
        if (!ptx::mbar_wait(ptx::smem_u32(&bar_full[stage]), phase, abort_p)) { ok = false; break; }
        ptx::tc_fence_after();
        const uint32_t a_src = smem_base + stage * Ck::STAGE, b_src = a_src + Ck::A_BYTES;
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; ++k) {
          const uint64_t adesc = ptx::smem_desc_sw128(a_src + k * (UMMA_K * 2), 16, 1024);
          const uint64_t bdesc = B_NK ? ptx::smem_desc_sw128(b_src + k * (UMMA_K * 2), 16, 1024)
                                      : ptx::smem_desc_sw128(b_src + k * (UMMA_K * 128), B_ATOM_BYTES, 1024);
          ptx::mma_bf16(tmem_base, adesc, bdesc, idesc, (kb | static_cast<uint32_t>(k)) != 0u);
        }
        ptx::mma_commit(ptx::smem_u32(&bar_empty[stage]));
        if (++stage == Ck::STAGES) { stage = 0; phase ^= 1u; }
      }
      if (ok && num_kb > 0) ptx::mma_commit(ptx::smem_u32(&bar_tmem_full));
    }
  } else {
    // ---------------- the accumulator of this range: TMEM -> this CTA's shared memory ----------------
    // Row r lies at r * 1 KB; its 16-byte chunk c at position c ^ (r & 7), so that the eight lanes of a store
    // wavefront (eight rows, the same c) fall into eight different bank groups. The ring below is drained: every
    // copy has landed and every MMA that read it has completed once bar_tmem_full has fired.
    const uint32_t e = static_cast<uint32_t>(warp) - 2u, quad = static_cast<uint32_t>(warp) & 3u, half = e >> 2;
    {  // the bias is fetched before the wait: its latency hides under the K loop
      const uint32_t gcol0 = tc.n * BN + static_cast<uint32_t>(lane) * 4u;
#pragma unroll
      for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int j = 0; j < 4; ++j)
          bv[h][j] = (bias != nullptr && gcol0 + 128u * h < N) ? __ldg(bias + gcol0 + 128u * h + j) : 0.0f;
    }
    bool ok = true;
    if (num_kb > 0) {
      ok = ptx::mbar_wait(ptx::smem_u32(&bar_tmem_full), 0u, abort_p);
      ptx::tc_fence_after();
    }
    {
      const uint32_t row = quad * 32u + static_cast<uint32_t>(lane);
      const uint32_t prow = smem_base + row * 1024u;
#pragma unroll 1
      for (uint32_t q = 0; q < 4; ++q) {
        uint32_t r[32];
        if (num_kb > 0 && ok) {
          ptx::tmem_ld_32x32(tmem_base + ((quad * 32u) << 16) + half * 128 + q * 32, r);
          ptx::tmem_ld_wait_for(r);
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = 0u;
        }
#pragma unroll
        for (uint32_t v = 0; v < 8; ++v) {
          const uint32_t chunk = half * 32u + q * 8u + v;
          ptx::st_shared_v4(prow + ((chunk ^ (row & 7u)) << 4), r[v * 4], r[v * 4 + 1], r[v * 4 + 2], r[v * 4 + 3]);
        }
      }
    }
    ptx::named_bar_sync(1, EPI_WARPS * 32);  // the whole plane is in shared memory
    // The rows other CTAs own go to the workspace: a warp per row, 512 contiguous bytes per store instruction.
    float* mine = ws + static_cast<size_t>(blockIdx.x) * (UMMA_M * BN);
    for (uint32_t row = e; row < rows_here; row += EPI_WARPS) {
      if (row / ROWS_PER == rank) continue;
#pragma unroll
      for (uint32_t h = 0; h < 2; ++h) {
        const uint32_t chunk = static_cast<uint32_t>(lane) + 32u * h;
        const float4 v = ld_shared_v4(smem_base + row * 1024u + ((chunk ^ (row & 7u)) << 4));
        __stcg(reinterpret_cast<float4*>(mine + row * BN + chunk * 4u), v);
      }
    }
  }

  // every range of the tile is in its CTA's shared memory or, for the rows other CTAs own, in the workspace: the
  // cluster barrier orders those writes before the peers' reads
  ptx::tc_fence_before();
  __syncthreads();  // the warps' roles have diverged: converge before the aligned cluster barrier
  ptx::cluster_arrive();
  ptx::cluster_wait();

  if (warp >= 2) {
    // ---------------- this CTA's rows of the tile: ranges in ascending order, bias, activation ----------------
    // A lane owns the 16-byte chunks `lane` and `lane + 32` of a row; R rows are in flight together.
    constexpr int R = KS <= 4 ? 4 : 2;
    const uint32_t e = static_cast<uint32_t>(warp) - 2u;
    const uint32_t r_lo = rank * ROWS_PER, r_hi = min(rows_here, r_lo + ROWS_PER);
    const uint32_t gcol0 = tc.n * BN + static_cast<uint32_t>(lane) * 4u;
    bool col_ok[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) col_ok[h] = gcol0 + 128u * h < N;  // N % 8 == 0: a group of four columns is inside or outside as a whole
    const float* peers = ws + static_cast<size_t>(tile) * KS * (UMMA_M * BN);
#pragma unroll 1
    for (uint32_t row0 = r_lo + e; row0 < r_hi; row0 += EPI_WARPS * R) {
      float4 p[R][KS][2];
#pragma unroll
      for (int i = 0; i < R; ++i) {
        const uint32_t row = row0 + EPI_WARPS * i;
#pragma unroll
        for (int r2 = 0; r2 < KS; ++r2) {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const uint32_t chunk = static_cast<uint32_t>(lane) + 32u * h;
            if (row >= r_hi || !col_ok[h]) p[i][r2][h] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            else if (static_cast<uint32_t>(r2) == rank) p[i][r2][h] = ld_shared_v4(smem_base + row * 1024u + ((chunk ^ (row & 7u)) << 4));
            else p[i][r2][h] = __ldcg(reinterpret_cast<const float4*>(peers + (static_cast<size_t>(r2) * UMMA_M + row) * BN + chunk * 4u));
          }
        }
      }
#pragma unroll
      for (int i = 0; i < R; ++i) {
        const uint32_t row = row0 + EPI_WARPS * i;
        if (row >= r_hi) continue;
        const size_t grow = static_cast<size_t>(tc.m) * UMMA_M + row;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          if (!col_ok[h]) continue;
          float f0 = 0.0f, f1 = 0.0f, f2 = 0.0f, f3 = 0.0f;
#pragma unroll
          for (int r2 = 0; r2 < KS; ++r2) {  // ascending ranges: ascending k, like the one-pass kernel
            f0 += p[i][r2][h].x; f1 += p[i][r2][h].y; f2 += p[i][r2][h].z; f3 += p[i][r2][h].w;
          }
          if constexpr (OUT_F32) {
            *reinterpret_cast<float4*>(c_f32 + grow * c_pitch + gcol0 + 128u * h) =
                make_float4(f0 * alpha, f1 * alpha, f2 * alpha, f3 * alpha);
          } else {
            f0 += bv[h][0]; f1 += bv[h][1]; f2 += bv[h][2]; f3 += bv[h][3];  // a sum is never -0: a zero bias keeps its bits
            if (act == TCAB_ACT_RELU) {
              f0 = fmaxf(f0, 0.0f); f1 = fmaxf(f1, 0.0f); f2 = fmaxf(f2, 0.0f); f3 = fmaxf(f3, 0.0f);
            }
            const __nv_bfloat162 h0 = __floats2bfloat162_rn(f0, f1), h1 = __floats2bfloat162_rn(f2, f3);
            *reinterpret_cast<uint2*>(c_raw + grow * N + gcol0 + 128u * h) =
                make_uint2(*reinterpret_cast<const uint32_t*>(&h0), *reinterpret_cast<const uint32_t*>(&h1));
          }
        }
      }
    }
  }

  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, UMMA_N);
  }
  if (threadIdx.x == 0 && abort_flag != 0) g_gemm_status = 5;
}

// Second pass of a K-split contraction: c = act(sum over ranges of partial + bias), bf16. Eight columns per thread.
__global__ void __launch_bounds__(256)
gemm_split_finish(const float* __restrict__ partial, const float* __restrict__ bias, __nv_bfloat16* __restrict__ c,
                  uint32_t M, uint32_t N, uint32_t ksplit, int act) {
  const size_t groups = static_cast<size_t>(M) * (N / 8);
  const size_t gidx = static_cast<size_t>(blockIdx.x) * 256 + threadIdx.x;
  if (gidx >= groups) return;
  const size_t off = gidx * 8, plane = static_cast<size_t>(M) * N;
  const uint32_t col = static_cast<uint32_t>(off % N);
  float f[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) f[j] = 0.0f;
  for (uint32_t ks = 0; ks < ksplit; ++ks) {  // ascending ranges: ascending k, like the one-pass kernel
    const float4 p0 = *reinterpret_cast<const float4*>(partial + ks * plane + off);
    const float4 p1 = *reinterpret_cast<const float4*>(partial + ks * plane + off + 4);
    f[0] += p0.x; f[1] += p0.y; f[2] += p0.z; f[3] += p0.w;
    f[4] += p1.x; f[5] += p1.y; f[6] += p1.z; f[7] += p1.w;
  }
  uint32_t w[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    float f0 = f[2 * j], f1 = f[2 * j + 1];
    if (bias != nullptr) {
      f0 += __ldg(bias + col + 2 * j);
      f1 += __ldg(bias + col + 2 * j + 1);
    }
    if (act == TCAB_ACT_RELU) {
      f0 = fmaxf(f0, 0.0f);
      f1 = fmaxf(f1, 0.0f);
    }
    const __nv_bfloat162 hh = __floats2bfloat162_rn(f0, f1);
    w[j] = *reinterpret_cast<const uint32_t*>(&hh);
  }
  *reinterpret_cast<uint4*>(c + off) = make_uint4(w[0], w[1], w[2], w[3]);
}

// Workspace of the K split: one buffer per (device, stream), grown on demand up to kSplitWorkspaceBytes.
constexpr size_t kSplitWorkspaceBytes = static_cast<size_t>(64) << 20;
constexpr size_t kSplitCounters = 16384;  // arrival counters of the fused fold: 64 KiB per (device, stream), zero between launches
float* gemm_split_workspace(cudaStream_t stream, size_t bytes) {
  if (bytes > kSplitWorkspaceBytes) return nullptr;
  return static_cast<float*>(stream_scratch(kScratchGemm, stream, bytes, true));
}

// cuTensorMapEncodeTiled through the runtime's driver entry point lookup: the library does not
// link libcuda, so it still loads (and reports TCAB_ERR_CUDA) on a box without a driver.
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn encode_fn() {
  static EncodeFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeFn>(p);
    else
      cudaGetLastError();
  });
  return fn;
}

// A 2-D bf16 row-major tensor [rows, cols] (cols contiguous) with a box of box_rows x box_cols columns:
// 64 columns (128-byte rows, 128-byte swizzle) or 32 columns (64-byte rows, 64-byte swizzle).
int make_map(CUtensorMap* m, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows, uint32_t box_cols = 64) {
  EncodeFn enc = encode_fn();
  if (enc == nullptr) return fail(TCAB_ERR_CUDA, "gemm_bias_act: cuTensorMapEncodeTiled is not available");
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {cols * 2};
  const cuuint32_t box[2] = {box_cols, box_rows};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, box_cols == 64 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(TCAB_ERR_CUDA, "gemm_bias_act: cuTensorMapEncodeTiled failed (%d)", static_cast<int>(r));
  return TCAB_OK;
}

// A 2-D fp32 row-major tensor with a box of box_rows x 32 columns (128-byte rows, 128-byte swizzle).
int make_map_f32(CUtensorMap* m, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows, uint32_t box_cols,
                 uint64_t pitch = 0) {  // pitch: elements between rows (0 = cols)
  EncodeFn enc = encode_fn();
  if (enc == nullptr) return fail(TCAB_ERR_CUDA, "chain_contract: cuTensorMapEncodeTiled is not available");
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {(pitch ? pitch : cols) * 4};
  const cuuint32_t box[2] = {box_cols, box_rows};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(base), dims, strides, box, elem,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(TCAB_ERR_CUDA, "chain_contract: cuTensorMapEncodeTiled failed (%d)", static_cast<int>(r));
  return TCAB_OK;
}

}  // namespace


int gemm_device_status(int* out) {
  if (cudaMemcpyFromSymbol(out, g_gemm_status, sizeof(int)) != cudaSuccess) {
    cudaGetLastError();
    return fail(TCAB_ERR_CUDA, "device_status: cannot read the status word");
  }
  return TCAB_OK;
}

// The cluster K-split kernel for a cluster of ks CTAs (2..8); the fp32-out forms exist for 2, 4 and 8.
const void* cluster_k_fn(int ks, int form = 0) {  // form: 0 bf16 out, 1 fp32 out with b [K, N], 2 fp32 out with b [N, K]
  if (form == 1) {
    switch (ks) {
      case 2: return reinterpret_cast<const void*>(gemm_cluster_k_kernel<2, true, false>);
      case 4: return reinterpret_cast<const void*>(gemm_cluster_k_kernel<4, true, false>);
      case 8: return reinterpret_cast<const void*>(gemm_cluster_k_kernel<8, true, false>);
      default: return nullptr;
    }
  }
  if (form == 2) {
    switch (ks) {
      case 2: return reinterpret_cast<const void*>(gemm_cluster_k_kernel<2, true, true>);
      case 4: return reinterpret_cast<const void*>(gemm_cluster_k_kernel<4, true, true>);
      case 8: return reinterpret_cast<const void*>(gemm_cluster_k_kernel<8, true, true>);
      default: return nullptr;
    }
  }
  switch (ks) {
    case 2: return reinterpret_cast<const void*>(gemm_cluster_k_kernel<2>);
    case 3: return reinterpret_cast<const void*>(gemm_cluster_k_kernel<3>);
    case 4: return reinterpret_cast<const void*>(gemm_cluster_k_kernel<4>);
    case 5: return reinterpret_cast<const void*>(gemm_cluster_k_kernel<5>);
    case 6: return reinterpret_cast<const void*>(gemm_cluster_k_kernel<6>);
    case 7: return reinterpret_cast<const void*>(gemm_cluster_k_kernel<7>);
    default: return reinterpret_cast<const void*>(gemm_cluster_k_kernel<8>);
  }
}

// How many clusters of ks CTAs of that kernel the current device holds at once (0 when it cannot say); asked once
// per device and size. The shared-memory attribute of the device's copy of the function is set on the way.
int cluster_k_resident(int ks, int form = 0) {
  constexpr int kMaxDev = 64;
  static std::mutex mu;
  static int cache_all[3][kMaxDev][9];  // 0 = not asked yet, -1 = none, else the count
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDev || ks < 2 || ks > 8 || form < 0 || form > 2) return 0;
  if (cluster_k_fn(ks, form) == nullptr) return 0;
  std::lock_guard<std::mutex> lock(mu);
  int (*cache)[9] = cache_all[form];
  if (cache[dev][ks] == 0) {
    const void* fn = cluster_k_fn(ks, form);
    int n = 0;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(ks) * 64);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = Ck::SMEM;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = static_cast<unsigned>(ks);
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(Ck::SMEM)) != cudaSuccess ||
        cudaOccupancyMaxActiveClusters(&n, fn, &cfg) != cudaSuccess) {
      cudaGetLastError();
      n = 0;
    }
    cache[dev][ks] = n > 0 ? n : -1;
  }
  return cache[dev][ks] > 0 ? cache[dev][ks] : 0;
}

int launch_gemm_bias_act(const __nv_bfloat16* a, const __nv_bfloat16* b, const float* bias, int act,
                         __nv_bfloat16* c, uint32_t m, uint32_t n, uint32_t k, cudaStream_t s) {
  if (m == 0 || n == 0) return TCAB_OK;
  const Tune& tn = tune(kGemm);
  // Which kernel: the 256 x 256 single-CTA kernel while its tiles fill the GPU; below that the double-buffered
  // kernels, whose 128-row tiles give twice the CTAs (measured 2048^3: 620 -> 820 TFLOP/s with CTA pairs, 905 with
  // single CTAs). tune p1 forces a kernel.
  int variant = tn.p1;
  if (variant == 5) variant = m <= 128 ? 3 : 4;  // the cluster K split where it applies, else what these shapes get
  if (variant <= 0 && k > 0) {
    const uint64_t tiles256 = static_cast<uint64_t>((m + BM - 1) / BM) * ((n + BN - 1) / BN);
    // (128 tiles on 148 SMs: the default is faster.) Single CTAs, not pairs: 2048^3 905 against 811 TFLOP/s,
    // 1024 x 4096 x 4096 863 against 826, 1024^3 the same
    if (2 * tiles256 <= static_cast<uint64_t>(sm_count())) variant = 3;
    // A tile count just above a whole number of rounds leaves the last round nearly empty (320 tiles on 148 SMs:
    // three rounds, 72 % of the CTA slots used). CTA pairs take a 256 x 256 tile per PAIR, so their rounds are half as
    // long and the count rounds up to a multiple of 74 instead of 148; their K loop runs at about 0.88 of the
    // single-CTA kernel's rate. Pairs where that trade pays (4000 x 5000 x 3000: 970 -> 1,100 TFLOP/s).
    else {
      const uint64_t sms = static_cast<uint64_t>(sm_count()), pairs = sms / 2;
      const double fill1 = static_cast<double>(tiles256) / static_cast<double>((tiles256 + sms - 1) / sms * sms);
      const double fill4 = static_cast<double>(tiles256) / static_cast<double>((tiles256 + pairs - 1) / pairs * pairs);
      if (pairs > 0 && fill4 * 0.88 > fill1 * 1.02) variant = 4;
    }
  }
  const bool default_kernel = !(variant == 3 || variant == 4 || (variant == 2 && k > 0));
  CUtensorMap ta, tb, tcm;
  {
    // the default kernel stores half boxes (32 x 32, 64-byte swizzle), the variants whole boxes (32 x 64)
    const int rc = make_map(&tcm, c, m, n, 32, default_kernel ? 32 : 64);
    if (rc != TCAB_OK) return rc;
  }
  if (k > 0) {
    int rc = make_map(&ta, a, m, k, BM);
    if (rc != TCAB_OK) return rc;
    rc = make_map(&tb, b, k, n, BK);
    if (rc != TCAB_OK) return rc;
  } else {
    // no K blocks: the kernel never touches the maps; encode them over c to keep them valid
    int rc = make_map(&ta, c, m, n, BM);
    if (rc != TCAB_OK) return rc;
    tb = ta;
  }
  // per launch, like the reference's launcher does above 48 KB (internal/cg/cxx/launch.go:145-155):
  // the attribute belongs to the current device's copy of the function
  const cudaError_t attr_err = cudaFuncSetAttribute(gemm_bias_act_kernel<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                    static_cast<int>(SMEM_BYTES));
  if (attr_err != cudaSuccess)
    return fail(TCAB_ERR_CUDA, "gemm_bias_act: cannot reserve %zu bytes of shared memory: %s", SMEM_BYTES,
                cudaGetErrorString(attr_err));
  // Few tiles and a long K: one cluster per 128 x 256 tile, one K range per CTA (gemm_cluster_k_kernel), as long as
  // every cluster is resident at once. tune p1 == 5 asks for it whatever the shape, p3 then gives the cluster size;
  // p2 == 32 keeps the two-launch workspace form below (p2 == 16 its one-launch variant).
  if (k > 0 && n % 8 == 0 && tn.p2 != 32 && tn.p2 != 16 && ((tn.p1 <= 0 && (variant == 3 || variant == 4) && tn.p3 <= 0) || tn.p1 == 5)) {
    const uint32_t all_kb = (k + BK - 1) / BK;
    const uint64_t tiles = static_cast<uint64_t>((m + UMMA_M - 1) / UMMA_M) * ((n + BN - 1) / BN);
    uint64_t ks = tn.p3 > 0 ? static_cast<uint64_t>(tn.p3) : static_cast<uint64_t>(sm_count()) / (tiles > 0 ? tiles : 1);
    if (tn.p3 <= 0 && ks > all_kb / 8) ks = all_kb / 8;    // at least eight K blocks (512 of K) per range
    if (ks > 8) ks = 8;                                     // the portable cluster size
    if (ks > all_kb) ks = all_kb;
    if (tn.p3 <= 0)
      while (ks >= 2 && static_cast<uint64_t>(cluster_k_resident(static_cast<int>(ks))) < tiles) --ks;  // one wave
    else if (ks >= 2 && cluster_k_resident(static_cast<int>(ks)) == 0)  // (the query also reserves the shared memory)
      ks = 0;
    float* ws = ks >= 2 ? gemm_split_workspace(s, static_cast<size_t>(tiles) * ks * Ck::PLANE_BYTES) : nullptr;
    if (ks >= 2 && ws != nullptr) {
      CUtensorMap ta2;
      const int rc = make_map(&ta2, a, m, k, UMMA_M);
      if (rc != TCAB_OK) return rc;
      const void* fn = cluster_k_fn(static_cast<int>(ks));
      uint32_t kb_per = (all_kb + static_cast<uint32_t>(ks) - 1) / static_cast<uint32_t>(ks);
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3(static_cast<unsigned>(tiles * ks));
      cfg.blockDim = dim3(THREADS);
      cfg.dynamicSmemBytes = Ck::SMEM;
      cfg.stream = s;
      cudaLaunchAttribute attr[1];
      attr[0].id = cudaLaunchAttributeClusterDimension;
      attr[0].val.clusterDim.x = static_cast<unsigned>(ks);
      attr[0].val.clusterDim.y = 1;
      attr[0].val.clusterDim.z = 1;
      cfg.attrs = attr;
      cfg.numAttrs = 1;
      float* c_f32 = nullptr;
      uint64_t c_pitch = 0;
      float alpha = 1.0f;
      void* args[] = {&ta2, &tb, &bias, &m, &n, &k, &act, &kb_per, &ws, &c, &c_f32, &c_pitch, &alpha};
      const cudaError_t le = cudaLaunchKernelExC(&cfg, fn, args);
      count_launch();
      if (le != cudaSuccess) {
        cudaGetLastError();
        return fail(TCAB_ERR_CUDA, "gemm_bias_act (cluster K split): launch failed: %s", cudaGetErrorString(le));
      }
      return TCAB_OK;
    }
  }
  if (variant == 3 || variant == 4) {
    // double-buffered accumulators: A boxes of 128 rows; variant 4 runs clusters of two CTAs
    const bool pair = variant == 4;
    CUtensorMap ta2;
    int rc = k > 0 ? make_map(&ta2, a, m, k, UMMA_M) : TCAB_OK;
    if (rc != TCAB_OK) return rc;
    if (k == 0) ta2 = ta;
    const size_t smem = pair ? Db<true>::SMEM : Db<false>::SMEM;
    const void* fn = pair ? reinterpret_cast<const void*>(gemm_bias_act_db_kernel<true>)
                          : reinterpret_cast<const void*>(gemm_bias_act_db_kernel<false>);
    const cudaError_t ae = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (ae != cudaSuccess)
      return fail(TCAB_ERR_CUDA, "gemm_bias_act: cannot reserve %zu bytes of shared memory: %s", smem,
                  cudaGetErrorString(ae));
    const uint32_t tile_m = pair ? Db<true>::TILE_M : Db<false>::TILE_M;
    const uint64_t tiles = static_cast<uint64_t>((m + tile_m - 1) / tile_m) * ((n + BN - 1) / BN);
    const uint64_t ctas_per_tile = pair ? 2 : 1;
    uint64_t groups = (tn.p0 > 0 ? static_cast<uint64_t>(tn.p0) : static_cast<uint64_t>(sm_count())) / ctas_per_tile;
    // Few tiles and a long K: the K blocks of a tile are cut into ranges, one unit of work each; the fp32
    // partials go to a workspace and gemm_split_finish adds them, the bias and the activation. tune p3 forces
    // the number of ranges.
    const uint32_t all_kb = (k + BK - 1) / BK;
    uint32_t ksplit = 1, kb_per = all_kb;
    float* partial = nullptr;
    uint32_t* counters = nullptr;
    if (k > 0 && n % 8 == 0) {
      uint64_t want = tn.p3 > 0 ? static_cast<uint64_t>(tn.p3) : (tiles > 0 ? groups / tiles : 1);
      if (tn.p3 <= 0 && want > all_kb / 16) want = all_kb / 16;  // at least sixteen K blocks (1024 of K) per range
      if (want > all_kb) want = all_kb;
      const size_t plane = static_cast<size_t>(m) * n * sizeof(float);
      if (want > kSplitWorkspaceBytes / plane) want = kSplitWorkspaceBytes / plane;
      if (want >= 2) {
        kb_per = (all_kb + static_cast<uint32_t>(want) - 1) / static_cast<uint32_t>(want);
        ksplit = (all_kb + kb_per - 1) / kb_per;  // no empty range
        partial = ksplit > 1 ? gemm_split_workspace(s, plane * ksplit) : nullptr;
        if (partial == nullptr) {
          ksplit = 1;
          kb_per = all_kb;
        }
        // The ranges are added by a second launch (gemm_split_finish). The one-launch form -- one counter per (tile,
        // CTA of the pair, epilogue warp), the last arriver folds -- is kept behind tune p2 == 16: it was measured
        // slower (128 x 8192 x 8192: 46 us against 39 us, 256 x 8192 x 4096: 37 against 31; equal from 64 tiles up),
        // because the few warps that arrive last do at the tail what the second launch spreads over every SM.
        if (ksplit > 1 && tn.p2 == 16 && tiles * ctas_per_tile * EPI_WARPS <= kSplitCounters)
          counters = static_cast<uint32_t*>(stream_scratch(kScratchGemmCounters, s, kSplitCounters * sizeof(uint32_t), false, true));
      }
    }
    const uint64_t units = tiles * ksplit;
    if (groups > units) groups = units;
    if (groups < 1) groups = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(ctas_per_tile * groups));
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = pair ? 2 : 1;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    void* args[] = {&ta2, &tb, &tcm, &bias, &m, &n, &k, &act, &ksplit, &kb_per, &partial, &counters, &c};
    const cudaError_t le = cudaLaunchKernelExC(&cfg, fn, args);
    count_launch();
    if (le != cudaSuccess) {
      cudaGetLastError();
      return fail(TCAB_ERR_CUDA, "gemm_bias_act (double-buffered): launch failed: %s", cudaGetErrorString(le));
    }
    if (ksplit > 1 && counters == nullptr) {
      const size_t groups8 = static_cast<size_t>(m) * (n / 8);
      gemm_split_finish<<<static_cast<unsigned>((groups8 + 255) / 256), 256, 0, s>>>(partial, bias, c, m, n, ksplit, act);
      count_launch();
      return check_launch("gemm_split_finish");
    }
    return TCAB_OK;
  }
  if (variant == 2 && k > 0) {
    // CTA pairs: A boxes of 128 rows, clusters of two CTAs
    CUtensorMap ta2;
    int rc = make_map(&ta2, a, m, k, UMMA_M);
    if (rc != TCAB_OK) return rc;
    const cudaError_t ae = cudaFuncSetAttribute(gemm_bias_act_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                static_cast<int>(P_SMEM_BYTES));
    if (ae != cudaSuccess)
      return fail(TCAB_ERR_CUDA, "gemm_bias_act: cannot reserve %zu bytes of shared memory: %s", P_SMEM_BYTES,
                  cudaGetErrorString(ae));
    const uint64_t ptiles = static_cast<uint64_t>((m + P_BM - 1) / P_BM) * ((n + BN - 1) / BN);
    uint64_t pairs = (tn.p0 > 0 ? static_cast<uint64_t>(tn.p0) : static_cast<uint64_t>(sm_count())) / 2;
    if (pairs > ptiles) pairs = ptiles;
    if (pairs < 1) pairs = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(2 * pairs));
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = P_SMEM_BYTES;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const cudaError_t le = cudaLaunchKernelEx(&cfg, gemm_bias_act_pair_kernel, ta2, tb, tcm, bias, m, n, k, act);
    count_launch();
    if (le != cudaSuccess) {
      cudaGetLastError();
      return fail(TCAB_ERR_CUDA, "gemm_bias_act (pairs): launch failed: %s", cudaGetErrorString(le));
    }
    return TCAB_OK;
  }
  const uint64_t tiles = static_cast<uint64_t>((m + BM - 1) / BM) * ((n + BN - 1) / BN);
  uint64_t grid = tn.p0 > 0 ? static_cast<uint64_t>(tn.p0) : static_cast<uint64_t>(sm_count());
  if (grid > tiles) grid = tiles;
  gemm_bias_act_kernel<false, false><<<static_cast<unsigned>(grid), THREADS, SMEM_BYTES, s>>>(ta, tb, tcm, bias, m, n, k, act, 1.0f);
  count_launch();
  return check_launch("gemm_bias_act_kernel");
}

// c[m, n] (fp32) = alpha * sum_k a[m, k] * b[k, n] (or b[n, k]) over bf16 operands, fp32 accumulation in the tensor
// cores: what a contraction chain with the plain product as its map, a sum reducer and init 0 asks for. The caller
// has checked the alignment rules (K % 8 == 0, N % 8 == 0 for [K, N] operands, N % 4 == 0, 16-byte aligned
// pointers).
int launch_contract_bf16_tc(const __nv_bfloat16* a, const __nv_bfloat16* b, int b_is_nk, float alpha, float* c, uint32_t m,
                            uint32_t n, uint32_t k, cudaStream_t s, uint64_t c_pitch) {
  // c_pitch: elements between the rows of c (0 = n): c may be a block of columns of a wider matrix
  if (m == 0 || n == 0) return TCAB_OK;
  if (k == 0) {  // an empty reduction: init = 0 everywhere
    const cudaError_t e = (c_pitch == 0 || c_pitch == n)
                              ? cudaMemsetAsync(c, 0, static_cast<size_t>(m) * n * sizeof(float), s)
                              : cudaMemset2DAsync(c, c_pitch * sizeof(float), 0, static_cast<size_t>(n) * sizeof(float), m, s);
    return e == cudaSuccess ? TCAB_OK : fail(TCAB_ERR_CUDA, "chain_contract: cudaMemsetAsync failed: %s", cudaGetErrorString(e));
  }
  // Few 256 x 256 tiles and a long K: one cluster per 128 x 256 tile, a K range per CTA (see gemm_cluster_k_kernel)
  {
    const uint64_t tiles256 = static_cast<uint64_t>((m + BM - 1) / BM) * ((n + BN - 1) / BN);
    const uint64_t tiles128 = static_cast<uint64_t>((m + UMMA_M - 1) / UMMA_M) * ((n + BN - 1) / BN);
    const uint32_t all_kb = (k + BK - 1) / BK;
    const int form = b_is_nk ? 2 : 1;
    if (2 * tiles256 <= static_cast<uint64_t>(sm_count()) && all_kb >= 16 && tune(kGemm).p2 != 32) {
      uint64_t ks = static_cast<uint64_t>(sm_count()) / tiles128;
      if (ks > all_kb / 8) ks = all_kb / 8;
      ks = ks >= 8 ? 8 : ks >= 4 ? 4 : ks >= 2 ? 2 : 0;
      while (ks >= 2 && static_cast<uint64_t>(cluster_k_resident(static_cast<int>(ks), form)) < tiles128) ks >>= 1;
      float* ws = ks >= 2 ? gemm_split_workspace(s, static_cast<size_t>(tiles128) * ks * Ck::PLANE_BYTES) : nullptr;
      if (ks >= 2 && ws != nullptr) {
        CUtensorMap ta2, tb2;
        int rc = make_map(&ta2, a, m, k, UMMA_M);
        if (rc == TCAB_OK) rc = b_is_nk ? make_map(&tb2, b, n, k, BN) : make_map(&tb2, b, k, n, BK);
        if (rc != TCAB_OK) return rc;
        const void* fn = cluster_k_fn(static_cast<int>(ks), form);
        uint32_t kb_per = (all_kb + static_cast<uint32_t>(ks) - 1) / static_cast<uint32_t>(ks);
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(static_cast<unsigned>(tiles128 * ks));
        cfg.blockDim = dim3(THREADS);
        cfg.dynamicSmemBytes = Ck::SMEM;
        cfg.stream = s;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = static_cast<unsigned>(ks);
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        const float* bias = nullptr;
        int act = TCAB_ACT_NONE;
        __nv_bfloat16* c_raw = nullptr;
        uint64_t pitch = c_pitch ? c_pitch : n;
        void* args[] = {&ta2, &tb2, &bias, &m, &n, &k, &act, &kb_per, &ws, &c_raw, &c, &pitch, &alpha};
        const cudaError_t le = cudaLaunchKernelExC(&cfg, fn, args);
        count_launch();
        if (le != cudaSuccess) {
          cudaGetLastError();
          return fail(TCAB_ERR_CUDA, "chain_contract (cluster K split): launch failed: %s", cudaGetErrorString(le));
        }
        return TCAB_OK;
      }
    }
  }
  CUtensorMap ta, tb, tcm;
  int rc = make_map(&ta, a, m, k, BM);
  if (rc == TCAB_OK) rc = b_is_nk ? make_map(&tb, b, n, k, BN) : make_map(&tb, b, k, n, BK);
  if (rc == TCAB_OK) rc = make_map_f32(&tcm, c, m, n, 32, 32, c_pitch);
  if (rc != TCAB_OK) return rc;
  const void* fn = b_is_nk ? reinterpret_cast<const void*>(gemm_bias_act_kernel<true, true>)
                           : reinterpret_cast<const void*>(gemm_bias_act_kernel<true, false>);
  const cudaError_t ae = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(SMEM_BYTES));
  if (ae != cudaSuccess)
    return fail(TCAB_ERR_CUDA, "chain_contract: cannot reserve %zu bytes of shared memory: %s", SMEM_BYTES, cudaGetErrorString(ae));
  const uint64_t tiles = static_cast<uint64_t>((m + BM - 1) / BM) * ((n + BN - 1) / BN);
  uint64_t grid = static_cast<uint64_t>(sm_count());
  if (grid > tiles) grid = tiles;
  const float* bias = nullptr;
  int act = TCAB_ACT_NONE;
  void* args[] = {&ta, &tb, &tcm, &bias, &m, &n, &k, &act, &alpha};
  const cudaError_t le = cudaLaunchKernel(fn, dim3(static_cast<unsigned>(grid)), dim3(THREADS), args, SMEM_BYTES, s);
  count_launch();
  if (le != cudaSuccess) {
    cudaGetLastError();
    return fail(TCAB_ERR_CUDA, "chain_contract (tensor cores): launch failed: %s", cudaGetErrorString(le));
  }
  return TCAB_OK;
}

// ------------------------------------------------------------------------------------------------------------
// fp32 contraction chains with the plain product on the tensor cores. x = x0 + x1 + x2 with three bf16 pieces
// (x0 = bf16(x), x1 = bf16(x - x0), x2 = bf16(x - x0 - x1): 24 significant bits, the remainder is below
// 2^-24 |x|). a * b = sum of nine piece products, of which the six with weight of at least 2^-16 are kept:
// a2 b0, a1 b1, a0 b2, a1 b0, a0 b1, a0 b0 (what is dropped is below 3 * 2^-24 |a b|). Written side by side
// along K -- A' = [a2 | a1 | a0 | a1 | a0 | a0] ([M, 6 K]) against B' = [b0; b1; b2; b0; b1; b0] ([6 K, N]) --
// they are ONE bf16 contraction with fp32 accumulation, which the kernel above already is; the smallest terms
// come first in K. Products of bf16 values are exact in fp32, so the error of an output is 2e-7 of sum |a||b|
// plus the accumulation's, against 6e-8 per operation for the scalar kernel.
// ------------------------------------------------------------------------------------------------------------
namespace {

constexpr size_t kSplit3WorkspaceBytes = static_cast<size_t>(512) << 20;

__device__ __forceinline__ void split3(float x, unsigned short* p) {
  const __nv_bfloat16 h0 = __float2bfloat16_rn(x);
  float r = x - __bfloat162float(h0);
  if (!(fabsf(x) <= 3.0e38f)) r = 0.0f;  // inf and NaN stay in the first piece alone
  const __nv_bfloat16 h1 = __float2bfloat16_rn(r);
  r -= __bfloat162float(h1);
  const __nv_bfloat16 h2 = __float2bfloat16_rn(r);
  p[0] = __bfloat16_as_ushort(h0);
  p[1] = __bfloat16_as_ushort(h1);
  p[2] = __bfloat16_as_ushort(h2);
}

// src [rows, cols] fp32 (cols % 4 == 0; `pitch` elements between its rows: it may be a block of columns of a wider
// matrix) -> dst bf16, contiguous: six blocks of pieces order[0..5], side by side ([rows, 6 cols], STACK = false) or
// below each other ([6 rows, cols], STACK = true). A thread takes four consecutive elements.
template <bool STACK>
__global__ void __launch_bounds__(256)
split3_kernel(const float* __restrict__ src, uint64_t pitch, unsigned short* __restrict__ dst, uint64_t rows, uint32_t cols,
              uint32_t order) {
  const uint64_t q = static_cast<uint64_t>(blockIdx.x) * 256 + threadIdx.x;  // group of four
  const uint64_t per_row = cols / 4;
  if (q >= rows * per_row) return;
  const uint64_t r = q / per_row;
  const uint32_t c = static_cast<uint32_t>(q - r * per_row) * 4;
  const float4 v = __ldcs(reinterpret_cast<const float4*>(src + r * pitch + c));
  unsigned short pc[4][3];
  split3(v.x, pc[0]);
  split3(v.y, pc[1]);
  split3(v.z, pc[2]);
  split3(v.w, pc[3]);
#pragma unroll
  for (uint32_t j = 0; j < 6; ++j) {
    const uint32_t w = (order >> (4 * j)) & 3u;
    const uint64_t at = STACK ? (static_cast<uint64_t>(j) * rows + r) * cols + c : (r * 6 + j) * static_cast<uint64_t>(cols) + c;
    const uint2 out = make_uint2(static_cast<uint32_t>(pc[0][w]) | (static_cast<uint32_t>(pc[1][w]) << 16),
                                 static_cast<uint32_t>(pc[2][w]) | (static_cast<uint32_t>(pc[3][w]) << 16));
    *reinterpret_cast<uint2*>(dst + at) = out;
  }
}

}  // namespace

int launch_contract_f32_split3(const float* a, const float* b, int b_is_nk, float alpha, float* c, uint32_t m, uint32_t n,
                               uint32_t k, cudaStream_t s) {
  // a problem worth three launches (few output tiles then share their K over the CTAs of a cluster), 16-byte rows
  const Tune& tn0 = tune(kGemm);  // p2 == 256: p3 = log2 of the smallest m * n * k that takes this path (sweeps)
  const uint64_t min_work = 1ull << (tn0.p2 == 256 && tn0.p3 > 0 ? tn0.p3 : 29);
  if (static_cast<uint64_t>(m) * n * k < min_work || k < 256 || k % 4 != 0 || n % 4 != 0 || (!b_is_nk && n % 8 != 0))
    return TCAB_ERR_UNSUPPORTED;
  if (!aligned16(a) || !aligned16(b) || !aligned16(c) || static_cast<uint64_t>(k) * 6 > 0xffffffffull) return TCAB_ERR_UNSUPPORTED;
  // The pieces of a block of mc rows of a and of a block of nc columns (rows, for [N, K]) of b fit the workspace at a
  // time: 12 k bytes per row or column. The whole problem when that is enough; otherwise blocks of multiples of
  // 256 (at least 1024 each way, so that a block product still has 16 tiles or more), b's block outermost.
  const uint64_t per_line = static_cast<uint64_t>(k) * 12;
  const Tune& tn = tune(kGemm);  // p2 == 128: p3 = the workspace cap in MiB (tests of the blocked form)
  const uint64_t cap = tn.p2 == 128 && tn.p3 > 0 ? static_cast<uint64_t>(tn.p3) << 20 : kSplit3WorkspaceBytes;
  const uint64_t lines = cap / per_line;  // rows of a plus columns of b that fit
  uint32_t mc = m, nc = n;
  if (static_cast<uint64_t>(m) + n + 64 > lines) {
    if (lines < 2048 + 64) return TCAB_ERR_UNSUPPORTED;  // K so long that not even 1024 x 1024 blocks fit
    const uint64_t half = ((lines - 64) / 2) & ~static_cast<uint64_t>(255);
    nc = n <= half ? n : static_cast<uint32_t>(half);
    const uint64_t left = (lines - 64 - nc) & ~static_cast<uint64_t>(255);
    mc = m <= left ? m : static_cast<uint32_t>(left);
  }
  const size_t bytes_a = ((static_cast<size_t>(mc) * per_line) + 255) & ~static_cast<size_t>(255);
  const size_t bytes_b = static_cast<size_t>(nc) * per_line;
  unsigned char* ws = static_cast<unsigned char*>(stream_scratch(kScratchSplit3, s, bytes_a + bytes_b, true));
  if (ws == nullptr) return TCAB_ERR_UNSUPPORTED;
  unsigned short* a3 = reinterpret_cast<unsigned short*>(ws);
  unsigned short* b3 = reinterpret_cast<unsigned short*>(ws + bytes_a);
  constexpr uint32_t kOrderA = 2u | (1u << 4) | (0u << 8) | (1u << 12) | (0u << 16) | (0u << 20);  // a2 a1 a0 a1 a0 a0
  constexpr uint32_t kOrderB = 0u | (1u << 4) | (2u << 8) | (0u << 12) | (1u << 16) | (0u << 20);  // b0 b1 b2 b0 b1 b0
  for (uint32_t n0 = 0; n0 < n; n0 += nc) {
    const uint32_t nn = n - n0 < nc ? n - n0 : nc;  // a multiple of 8 (of 4 for [N, K]): n, n0 and nc are
    if (b_is_nk) {  // [N, K]: rows n0 .. n0 + nn, blocks side by side, like a's
      const uint64_t qb = static_cast<uint64_t>(nn) * (k / 4);
      split3_kernel<false><<<static_cast<unsigned>((qb + 255) / 256), 256, 0, s>>>(b + static_cast<size_t>(n0) * k, k, b3, nn, k, kOrderB);
    } else {        // [K, N]: columns n0 .. n0 + nn of every row, blocks below each other
      const uint64_t qb = static_cast<uint64_t>(k) * (nn / 4);
      split3_kernel<true><<<static_cast<unsigned>((qb + 255) / 256), 256, 0, s>>>(b + n0, n, b3, k, nn, kOrderB);
    }
    count_launch();
    for (uint32_t m0 = 0; m0 < m; m0 += mc) {
      const uint32_t mm = m - m0 < mc ? m - m0 : mc;
      if (n0 == 0 || mc < m) {  // a's pieces are still there when one block holds all of a
        const uint64_t qa = static_cast<uint64_t>(mm) * (k / 4);
        split3_kernel<false><<<static_cast<unsigned>((qa + 255) / 256), 256, 0, s>>>(a + static_cast<size_t>(m0) * k, k, a3, mm, k, kOrderA);
        count_launch();
      }
      int rc = check_launch("split3_kernel");
      if (rc == TCAB_OK)
        rc = launch_contract_bf16_tc(reinterpret_cast<const __nv_bfloat16*>(a3), reinterpret_cast<const __nv_bfloat16*>(b3), b_is_nk,
                                     alpha, c + static_cast<size_t>(m0) * n + n0, mm, nn, 6 * k, s, n);
      if (rc != TCAB_OK) return rc;
    }
  }
  return TCAB_OK;
}

}  // namespace tcab
