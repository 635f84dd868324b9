/*
 * tcab_tuning.h -- benchmarking and test hooks of libtcab.so. NOT part of the surface a host binds:
 * include/tcab.h does not include this file, results never depend on anything declared here beyond
 * the order in which partial results are folded, and the hooks are process-global and not
 * thread-safe (set them before the threads that launch are started). The reference has no
 * counterpart: its launch geometry is fixed when a kernel is emitted
 * (internal/cg/cxx/emit.go:203-239 deriveLaunch).
 */
#ifndef TCAB_TUNING_H_
#define TCAB_TUNING_H_

#include "tcab.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Overrides the heuristic launch shape of one kernel
 * family for this process. Values <= 0 restore the heuristic. Meant for benchmarking sweeps and for
 * tests that must reach every kernel variant; results never depend on it beyond the fold order.
 *   "softmax", "layernorm": p0 = threads per row, p1 = vectors per thread (layernorm, with p0 <= 0: 8 = the
 *       shared-memory kernel without its gamma / beta prefetch), p2 = CTAs per SM (persistent
 *       grid; for a forced layernorm cluster: vectors per thread 4, 8; softmax clusters: 8 or 16 vectors per
 *       thread), p3 = variant (softmax: 1 no cluster
 *       kernel, 2 always, 3 the shared-memory kernel, 6 no 16-byte vectors for rows that are not a multiple of
 *       four columns; layernorm: 1 gamma/beta in registers, 2 no cluster kernel,
 *       3 always, 4 the shared-memory kernel, 6 no 16-byte vectors for rows that are not whole vectors).
 *   "reduce_inner" (tcab_chain_reduce): p0 = threads per row (1, 4, 32, 256; middle-axis reductions: 32 = a warp per
 *       column tile whatever the shape), p1 = CTAs per row of the
 *       split path, p2 = 2 launches without programmatic dependent launch, 3 no 1024-thread CTAs for small problems, p3 = CTAs sharing the k axis of a
 *       middle-axis reduction (any value, 1 included, also keeps the kernel with a CTA per column tile where the
 *       library would take a warp per tile).
 *   "reduce_outer": p0 = vectors per lane (1, 2), p1 = warps splitting k (4, 8, 16; 1 = a warp per column tile
 *       whatever the shape), p2 = CTAs per SM,
 *       p3 = CTAs sharing the k axis (any of p0, p1, p3 keeps the kernel with a CTA per column tile).
 *   "gemm": p0 = CTAs of the persistent grid, p1 = kernel of tcab_gemm_bias_act (2 CTA pairs with
 *       512 x 256 tiles, 3 double-buffered accumulators on 128 x 256 tiles, 4 the same on CTA pairs, 5 one
 *       cluster per 128 x 256 tile with a K range per CTA, whatever the shape),
 *       p2 = outputs per thread and side of tcab_chain_contract's tile (4: 64 x 64 tiles, 8: 128 x 128; for
 *       tcab_gemm_bias_act 32: the K ranges go to a workspace and a second launch adds them, never the cluster
 *       form; 16: the same with the last-arriving epilogue warps adding them instead of the second launch;
 *       64: tcab_chain_contract keeps product chains (bf16, or large f32) on the scalar kernel instead of the
 *       tensor cores; 128: p3 = workspace cap in MiB of the three-piece f32 contraction, which then runs in blocks),
 *       p3 = ranges the K blocks of a tile are cut into by kernels 3, 4 and 5 (1 = no split; 2..8 for 5). */
TCAB_API int tcab_tune(const char* family, int p0, int p1, int p2, int p3);


/* The launcher's plan for a middle-axis chain reduction whose k axis may be cut over several CTAs
 * (few column tiles, long k): pure arithmetic, no device needed. Inputs: the number of (batch, column tile)
 * pairs, of output cells, the reduced extent, how many CTAs are resident on the whole GPU at once, the SM
 * count, and a forced number of ranges (0 = the heuristic). Outputs: the number of k ranges and their
 * length. Every range r covers [r * klen, min(nk, (r + 1) * klen)) and none is empty. */
TCAB_API int tcab_plan_outer_split(uint64_t tiles, uint64_t cells, uint32_t nk, uint64_t resident_ctas, int sms,
                                   int forced, uint32_t* ranges, uint32_t* klen);

/* The launchers' shape rules that are pure arithmetic, for tests without a device:
 *   outer_flat_g   - middle-axis reduction over [rows_or_batches, nk, nc]: column groups per tile when a warp takes a
 *                    (b, column tile) instead of a CTA (0 = a CTA per tile); groups of four columns when nc is a
 *                    multiple of four (aligned operands assumed), of one column otherwise;
 *   stream_cluster - CTAs per row of a streaming cluster for a row of nvec vectors at per_step vectors per CTA and step;
 *   rows32         - warps per CTA of the thread-per-row kernel for rows of nvec vectors and n_in operands (its shared
 *                    memory stays within 48 KiB; fewer than 2: not used). */
TCAB_API int tcab_plan_row_kernels(uint64_t rows_or_batches, uint32_t nk, uint32_t nc, int sms, uint32_t nvec,
                                   uint32_t per_step, int prefer_three, int n_in, uint32_t* outer_flat_g,
                                   uint32_t* stream_cluster, uint32_t* rows32);

/* The warp-per-(b, column tile) kernels of a middle-axis reduction over [batches, nk, nc] (pure arithmetic): the column
 * groups per tile (0 = those kernels are not used), and into how many ranges of klen rows the k axis is cut when
 * there are few narrow tiles and a long reduced axis (column statistics of a tall matrix). A CTA of eight warps takes
 * a range and leaves one partial result per output cell. Range r covers [r * klen, min(nk, (r + 1) * klen)), none
 * is empty, and batches * nc * ranges stays within max_partials. */
TCAB_API int tcab_plan_outer_flat_ranges(uint64_t batches, uint32_t nk, uint32_t nc, int sms, uint64_t max_partials,
                                         uint32_t* groups, uint32_t* ranges, uint32_t* klen);

/* The register-row kernel shape the softmax (op 0, fp32) and layer-norm (op 1, elem_bytes 2 or 4) launchers ask for on
 * aligned rows of nvec 16-byte vectors: threads per row and vector slots per thread, 0 / 0 when no compiled shape
 * holds the row. Pure arithmetic. Other kernels (shared-memory rows, clusters) may still take the row. */
TCAB_API int tcab_plan_row_shape(int op, int elem_bytes, uint32_t nvec, uint32_t* threads_per_row,
                                 uint32_t* slots_per_thread);

/* Validates a chain exactly as tcab_chain_prepare does and runs the run-time compiler on it for sm_100a, but
 * loads nothing: works on a host without a GPU (needs libnvrtc). A chain that has an ahead-of-time kernel is
 * compiled all the same. Arguments as tcab_chain_prepare, plus the bit masks of the operands that have one
 * value per row / one row shared by all rows / (middle-axis reductions) one value per output cell -- what the
 * entry points derive from the operands' shapes. */
TCAB_API int tcab_compile_check(const tcab_chain* chain, const int32_t* in_dtypes, uint32_t n_ins, int use,
                                int out_dtype, int row_value_mask, int shared_row_mask, int cell_value_mask);

#ifdef __cplusplus
}
#endif

#endif /* TCAB_TUNING_H_ */
