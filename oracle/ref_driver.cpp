// ref_driver.cpp -- runs the REFERENCE's own runtime primitives on the host.
//
// TEST INFRASTRUCTURE ONLY (see tcab_oracle.c). This file holds no arithmetic
// of its own beyond the map lambdas: every access goes through the reference's
// tca::rt::TensorView (bounds-predicated Get/Set, runtime/tca/view.h:77-127),
// every walk through its SeqIterator/CtaIterator/ThrIterator
// (runtime/tca/iterator.h:39-93) and every fold through its SeqReducer or the
// host branch of its WarpReducer (runtime/tca/reducer.h:36-57, 81-181). The
// reference's headers compile for the host through their own shim
// (runtime/tca/mapping.h:26-30), the way runtime/tests/cpu_tests.cpp uses them.
// It is built against the headers where they lie in the reference checkout
// (oracle/Makefile); the output goes to oracle/_ref/ and is never committed.
//
// Purpose: pin the oracle's reduction protocol (init, ascending fold, padded
// points read as 0, one Combine per output) bit-for-bit against the reference.
#include <cmath>
#include <cstdint>

#include "tca/iterator.h"
#include "tca/mapping.h"
#include "tca/reducer.h"
#include "tca/view.h"

namespace {

float CombineAdd(float a, float b) { return a + b; }
float CombineMax(float a, float b) { return fmaxf(a, b); }

}  // namespace

extern "C" {

// Row sums with the loop nest of the emitted one-tier reduce kernel
// (internal/cg/cxx/testdata/reduce_warp.cu:12-62): CTA-strided row tiles of
// `tile_rows`, one thread per row inside a tile, the reduced axis walked in
// sequential tiles of `tile_cols` with a saturating tail, SeqReducer brackets.
// Every (cta, thread) pair of the launch is visited in turn on the host.
void ref_row_sum_one_tier(const float* lhs, uint32_t d0, uint32_t d1, uint32_t ctas,
                          uint32_t threads, uint32_t tile_cols, float* out) {
  using namespace tca::rt;
  TensorView<const float, 2u> lhs_v(lhs, d0, d1);
  TensorView<float, 1u> out_v(out, d0);
  KernelInfo kinfo(ctas, threads);
  const unsigned tile_rows = threads;
  for (unsigned cta = 0u; cta < ctas; ++cta) {
    GridMapping grid_map(kinfo, 1u, ctas < 2u ? 2u : ctas);
    grid_map.set_linear_id(cta);
    for (unsigned tid = 0u; tid < threads; ++tid) {
      ThreadMapping thread_map(kinfo, 0u);
      thread_map.set_linear_id(tid);
      SeqReducer<float> reducer(0.0f, CombineAdd);
      const unsigned first = grid_map.index() * tile_rows;
      for (auto it0 = CtaIterator(grid_map, 0u, ctas, 0u, ctas * tile_rows, d0); it0.Has();
           it0.Next()) {
        const unsigned base = first + it0.Index();
        const unsigned left = d0 - umin(base, d0);
        const unsigned rows_here = umin(tile_rows, left);
        for (auto it1 = ThrIterator(thread_map, 0u, tile_rows, thread_map.index(), threads,
                                    rows_here);
             it1.Has(); it1.Next()) {
          reducer.Init();
          for (auto it2 = SeqIterator(0u, tile_cols, d1); it2.Has(); it2.Next()) {
            const unsigned span = umin(tile_cols, d1 - umin(it2.Index(), d1));
            for (auto it3 = SeqIterator(0u, 1u, span); it3.Has(); it3.Next()) {
              reducer.Reduce(lhs_v.Get(base + it1.Index(), it2.Index() + it3.Index()));
            }
          }
          out_v.Set(reducer.Combine(), base + it1.Index());
        }
      }
    }
  }
}

// Middle-axis map+reduce through the reference primitives, the class of the
// suite's row_sum / softmax kernels (testing/kernels/runtime/row_sum.tca:18-33):
// out[i,j] = fold_k f(x[i,k,j], z[i,k,j]). `pad_k` extra padded iterations are
// walked past the end of the reduced axis: TensorView::Get suppresses them to
// 0, which is how the reference's guarded tiles behave; lambda 0 = x*z,
// 1 = expf(x)*z. The additive fold is unaffected by the padded zeros only
// because 0 is read for BOTH operands (0*0 and expf(0)*0 are 0).
void ref_reduce_middle(const float* x, const float* z, uint32_t d0, uint32_t dk, uint32_t dc,
                       int lambda, uint32_t pad_k, float* out) {
  using namespace tca::rt;
  TensorView<const float, 3u> x_v(x, d0, dk, dc);
  TensorView<const float, 3u> z_v(z, d0, dk, dc);
  TensorView<float, 2u> out_v(out, d0, dc);
  SeqReducer<float> reducer(0.0f, CombineAdd);
  for (unsigned i = 0u; i < d0; ++i) {
    for (unsigned j = 0u; j < dc; ++j) {
      reducer.Init();
      for (auto it = SeqIterator(0u, 1u, dk + pad_k); it.Has(); it.Next()) {
        const float v = x_v.Get(i, it.Index(), j);
        const float w = z_v.Get(i, it.Index(), j);
        reducer.Reduce(lambda == 0 ? v * w : expf(v) * w);
      }
      out_v.Set(reducer.Combine(), i, j);
    }
  }
}

// A bare fold of n values: op 0 = add, 1 = fmaxf, through SeqReducer
// (kind 0) or the host branch of WarpReducer (kind 1), which the reference
// defines as the same sequential algebra (runtime/tca/reducer.h:133-135).
float ref_fold(const float* v, uint32_t n, int op, float init, int kind) {
  using namespace tca::rt;
  float (*fn)(float, float) = op == 0 ? CombineAdd : CombineMax;
  if (kind == 0) {
    SeqReducer<float> r(init, fn);
    r.Init();
    for (uint32_t i = 0; i < n; ++i) r.Reduce(v[i]);
    return r.Combine();
  }
  KernelInfo kinfo(1u, 32u);
  ThreadMapping tm(kinfo, 0u);
  float slot[1] = {0.0f};
  SmemView<float, 1u> staging(slot, 1u);
  WarpReducer<float> r(init, fn, tm, staging);
  r.Init();
  for (uint32_t i = 0; i < n; ++i) r.Reduce(v[i]);
  return r.Combine();
}

}  // extern "C"
