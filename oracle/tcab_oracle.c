/*
 * tcab_oracle.c -- CPU restatement of the reference's numeric CPU loops.
 *
 * TEST INFRASTRUCTURE ONLY. Nothing in the product path (the CUDA library, the
 * host builder, the Python package) may call, link or import this file. It is
 * the checker the parity tests compare the CUDA kernels against, and the thing
 * the benchmark times as its CPU baseline.
 *
 * The reference (dianpeng/tcacomp) has no numeric evaluator of its own IR. Its
 * expected values are recomputed at test time by naive loops with one shape:
 * an fp32 accumulator, the reduced index ascending, `acc = acc (+) v`, one
 * output at a time. Those loops live in
 *   - internal/e2e/e2e_test.go:228-240          (row sum)
 *   - internal/e2e/frontend_test.go:194-209     (matmul + piped scale)
 *   - testing/runners/<kernel>.cu main()        (14 suite kernels)
 *   - runtime/tca/reducer.h:36-57               (SeqReducer: Init/Reduce/Combine)
 * and every function below follows one of them, cited at the function.
 *
 * Pinning: the 14 suite kernels and the row-sum/matmul-scale cases are pinned
 * by the reference's own formulas (input formula elem(i), shapes, scalar
 * values, loop bodies). The reduction protocol (init, ascending fold,
 * out-of-range reads yield 0) is additionally checked bit-for-bit against the
 * reference's runtime headers compiled for the host (oracle/ref_driver.cpp).
 * The five benchmark configurations (map+row-reduce, row softmax, layer-norm,
 * outer-axis sum/max/argmax, bf16 contraction with bias+ReLU) have no stored
 * expected outputs in the reference: for those, PARITY IS UNPINNED by the
 * reference beyond "a naive sequential-fp32 loop in the reference's style on
 * identical inputs"; their formulas come from the benchmark definition.
 *
 * Numeric policy (design/syntax-design.md:601-607): IEEE per operation, no
 * fast-math, bf16 is a storage type with fp32 arithmetic. This file is built
 * with -ffp-contract=off so that no FMA contraction happens on the CPU side.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <string.h>

#include <pthread.h>
#include <stdlib.h>
#include <unistd.h>

#define ORC_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------------ */
/* helpers                                                                    */
/* ------------------------------------------------------------------------ */

/* Row-parallel driver. The independent axis (rows / batch / M) is cut into
 * contiguous blocks, one per thread; the arithmetic of each output, and so
 * every result bit, is the same for any thread count. (This image has no
 * OpenMP runtime, hence pthreads.) */
static int g_threads = 0;

ORC_API int orc_num_threads(void) {
  if (g_threads <= 0) {
    long n = sysconf(_SC_NPROCESSORS_ONLN);
    g_threads = n > 0 ? (int)n : 1;
  }
  return g_threads;
}

ORC_API void orc_set_num_threads(int n) {
  if (n > 0) g_threads = n;
}

typedef void (*orc_body)(const void* ctx, int64_t lo, int64_t hi);
typedef struct {
  orc_body body;
  const void* ctx;
  int64_t lo, hi;
} orc_task;

static void* orc_thread_main(void* p) {
  orc_task* t = (orc_task*)p;
  t->body(t->ctx, t->lo, t->hi);
  return NULL;
}

static void parallel_rows(int64_t n, orc_body body, const void* ctx) {
  int nt = orc_num_threads();
  if (nt > n) nt = (int)(n > 0 ? n : 1);
  if (nt <= 1) {
    body(ctx, 0, n);
    return;
  }
  pthread_t* th = (pthread_t*)malloc(sizeof(pthread_t) * (size_t)nt);
  orc_task* tk = (orc_task*)malloc(sizeof(orc_task) * (size_t)nt);
  for (int i = 0; i < nt; ++i) {
    tk[i].body = body;
    tk[i].ctx = ctx;
    tk[i].lo = n * i / nt;
    tk[i].hi = n * (i + 1) / nt;
    if (pthread_create(&th[i], NULL, orc_thread_main, &tk[i]) != 0) {
      body(ctx, tk[i].lo, tk[i].hi); /* could not spawn: run the block here */
      th[i] = (pthread_t)0;
      tk[i].body = NULL;
    }
  }
  for (int i = 0; i < nt; ++i)
    if (tk[i].body) pthread_join(th[i], NULL);
  free(th);
  free(tk);
}

/* bf16 <-> f32. bf16 is the top 16 bits of an IEEE binary32; conversion to
 * bf16 rounds to nearest even (what __float2bfloat16_rn does on the device). */
static inline float bf16_to_f32(uint16_t h) {
  uint32_t u = ((uint32_t)h) << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

static inline uint16_t f32_to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u); /* quiet NaN */
  uint32_t lsb = (u >> 16) & 1u;
  u += 0x7fffu + lsb;
  return (uint16_t)(u >> 16);
}

ORC_API void orc_f32_to_bf16(const float* src, uint16_t* dst, uint64_t n) {
  for (uint64_t i = 0; i < n; ++i) dst[i] = f32_to_bf16(src[i]);
}

ORC_API void orc_bf16_to_f32(const uint16_t* src, float* dst, uint64_t n) {
  for (uint64_t i = 0; i < n; ++i) dst[i] = bf16_to_f32(src[i]);
}

/* The reference's deterministic input formula, u32 wraparound included:
 * testing/runners/common.cuh:19-21 and internal/e2e/e2e_test.go:194-200. */
static inline float elem(uint32_t i) {
  return (float)((i * 2654435761u) % 1000u) / 1000.0f;
}

ORC_API void orc_elem_fill(float* dst, uint32_t n) {
  for (uint32_t i = 0; i < n; ++i) dst[i] = elem(i);
}

/* rsqrtf is a CUDA builtin the reference's runners call on the host through
 * nvcc (testing/runners/layernorm.cu:53); on the host it is 1/sqrtf(x). */
static inline float host_rsqrtf(float x) { return 1.0f / sqrtf(x); }

/* ------------------------------------------------------------------------ */
/* benchmark configurations                                                   */
/* ------------------------------------------------------------------------ */

/* Fused map + innermost-axis reduce: y[i] = sum_j (0.5*x[i,j] + 0.25)^2.
 * Loop shape: internal/e2e/e2e_test.go:228-240 (fp32 acc, columns ascending);
 * the map is applied per element before the fold, as SeqReducer::Reduce is fed
 * (runtime/tca/reducer.h:45-51). */
typedef struct {
  const float* x;
  uint32_t rows;
  uint32_t cols;
  float a;
  float b;
  float* y;
} orc_map_rowsum_affine_sq_ctx;

static void orc_map_rowsum_affine_sq_body(const void* p, int64_t lo, int64_t hi) {
  const orc_map_rowsum_affine_sq_ctx* q__ = (const orc_map_rowsum_affine_sq_ctx*)p;
  const float* x = q__->x;
  uint32_t rows = q__->rows;
  uint32_t cols = q__->cols;
  float a = q__->a;
  float b = q__->b;
  float* y = q__->y;
  (void)x;
  (void)rows;
  (void)cols;
  (void)a;
  (void)b;
  (void)y;
  for (int64_t r = lo; r < hi; ++r) {
    const float* xr = x + (size_t)r * cols;
    float acc = 0.0f;
    for (uint32_t c = 0; c < cols; ++c) {
      const float t = a * xr[c] + b;
      acc += t * t;
    }
    y[r] = acc;
  }
}

ORC_API void orc_map_rowsum_affine_sq(const float* x, uint32_t rows, uint32_t cols, float a, float b, float* y) {
  const orc_map_rowsum_affine_sq_ctx ctx__ = {x, rows, cols, a, b, y};
  parallel_rows((int64_t)rows, orc_map_rowsum_affine_sq_body, &ctx__);
}

/* Same in fp64, for attributing an error to the GPU or to the fp32 fold. */
typedef struct {
  const float* x;
  uint32_t rows;
  uint32_t cols;
  float a;
  float b;
  double* y;
} orc_map_rowsum_affine_sq_f64_ctx;

static void orc_map_rowsum_affine_sq_f64_body(const void* p, int64_t lo, int64_t hi) {
  const orc_map_rowsum_affine_sq_f64_ctx* q__ = (const orc_map_rowsum_affine_sq_f64_ctx*)p;
  const float* x = q__->x;
  uint32_t rows = q__->rows;
  uint32_t cols = q__->cols;
  float a = q__->a;
  float b = q__->b;
  double* y = q__->y;
  (void)x;
  (void)rows;
  (void)cols;
  (void)a;
  (void)b;
  (void)y;
  for (int64_t r = lo; r < hi; ++r) {
    const float* xr = x + (size_t)r * cols;
    double acc = 0.0;
    for (uint32_t c = 0; c < cols; ++c) {
      const double t = (double)a * (double)xr[c] + (double)b;
      acc += t * t;
    }
    y[r] = acc;
  }
}

ORC_API void orc_map_rowsum_affine_sq_f64(const float* x, uint32_t rows, uint32_t cols, float a, float b, double* y) {
  const orc_map_rowsum_affine_sq_f64_ctx ctx__ = {x, rows, cols, a, b, y};
  parallel_rows((int64_t)rows, orc_map_rowsum_affine_sq_f64_body, &ctx__);
}

/* Plain row reductions in the same loop shape (e2e_test.go:228-240), with the
 * reducers the builder can express: `acc + v`, `fmaxf(acc, v)`, `fminf(acc, v)`
 * (internal/ir/builtins.go:25-39). An empty row yields init (design/tca.md:299). */
typedef struct {
  const float* x;
  uint32_t rows;
  uint32_t cols;
  int op;
  float init;
  float* y;
} orc_row_reduce_ctx;

static void orc_row_reduce_body(const void* p, int64_t lo, int64_t hi) {
  const orc_row_reduce_ctx* q__ = (const orc_row_reduce_ctx*)p;
  const float* x = q__->x;
  uint32_t rows = q__->rows;
  uint32_t cols = q__->cols;
  int op = q__->op;
  float init = q__->init;
  float* y = q__->y;
  (void)x;
  (void)rows;
  (void)cols;
  (void)op;
  (void)init;
  (void)y;
  for (int64_t r = lo; r < hi; ++r) {
    const float* xr = x + (size_t)r * cols;
    float acc = init;
    for (uint32_t c = 0; c < cols; ++c) {
      const float v = xr[c];
      acc = op == 0 ? acc + v : (op == 1 ? fmaxf(acc, v) : fminf(acc, v));
    }
    y[r] = acc;
  }
}

ORC_API void orc_row_reduce(const float* x, uint32_t rows, uint32_t cols, int op, float init, float* y) {
  const orc_row_reduce_ctx ctx__ = {x, rows, cols, op, init, y};
  parallel_rows((int64_t)rows, orc_row_reduce_body, &ctx__);
}

/* Row softmax as a map|reduce|map chain: m = max_j x, s = sum_j expf(x - m),
 * y = expf(x - m) / s. Each reduction is the sequential fold of
 * runtime/tca/reducer.h:45-51; expf is libm's, as the reference's runner calls
 * it on the host (testing/runners/softmax.cu:53). The max fold starts from
 * -inf; an empty row writes nothing. */
typedef struct {
  const float* x;
  uint32_t rows;
  uint32_t cols;
  float* y;
} orc_softmax_rows_ctx;

static void orc_softmax_rows_body(const void* p, int64_t lo, int64_t hi) {
  const orc_softmax_rows_ctx* q__ = (const orc_softmax_rows_ctx*)p;
  const float* x = q__->x;
  uint32_t rows = q__->rows;
  uint32_t cols = q__->cols;
  float* y = q__->y;
  (void)x;
  (void)rows;
  (void)cols;
  (void)y;
  for (int64_t r = lo; r < hi; ++r) {
    const float* xr = x + (size_t)r * cols;
    float* yr = y + (size_t)r * cols;
    float m = -INFINITY;
    for (uint32_t c = 0; c < cols; ++c) m = fmaxf(m, xr[c]);
    float s = 0.0f;
    for (uint32_t c = 0; c < cols; ++c) s += expf(xr[c] - m);
    for (uint32_t c = 0; c < cols; ++c) yr[c] = expf(xr[c] - m) / s;
  }
}

ORC_API void orc_softmax_rows(const float* x, uint32_t rows, uint32_t cols, float* y) {
  const orc_softmax_rows_ctx ctx__ = {x, rows, cols, y};
  parallel_rows((int64_t)rows, orc_softmax_rows_body, &ctx__);
}

/* Layer-norm over bf16 rows with fp32 statistics and bf16 output:
 * mean = (sum_j x)/n; var = (sum_j (x-mean)^2)/n; y = (x-mean)/sqrtf(var+eps)*gamma+beta.
 * Loop shape: testing/runners/layernorm.cu:47-58 (map | reduce | map over the
 * innermost axis, fp32 acc ascending); bf16 operands are widened to fp32
 * before any arithmetic (design/syntax-design.md:601-607). */
typedef struct {
  const uint16_t* x;
  const uint16_t* gamma;
  const uint16_t* beta;
  uint32_t rows;
  uint32_t cols;
  float eps;
  uint16_t* y;
} orc_layernorm_rows_bf16_ctx;

static void orc_layernorm_rows_bf16_body(const void* p, int64_t lo, int64_t hi) {
  const orc_layernorm_rows_bf16_ctx* q__ = (const orc_layernorm_rows_bf16_ctx*)p;
  const uint16_t* x = q__->x;
  const uint16_t* gamma = q__->gamma;
  const uint16_t* beta = q__->beta;
  uint32_t rows = q__->rows;
  uint32_t cols = q__->cols;
  float eps = q__->eps;
  uint16_t* y = q__->y;
  (void)x;
  (void)gamma;
  (void)beta;
  (void)rows;
  (void)cols;
  (void)eps;
  (void)y;
  for (int64_t r = lo; r < hi; ++r) {
    const uint16_t* xr = x + (size_t)r * cols;
    uint16_t* yr = y + (size_t)r * cols;
    float s = 0.0f;
    for (uint32_t c = 0; c < cols; ++c) s += bf16_to_f32(xr[c]);
    const float mean = s / (float)cols;
    float q = 0.0f;
    for (uint32_t c = 0; c < cols; ++c) {
      const float d = bf16_to_f32(xr[c]) - mean;
      q += d * d;
    }
    const float var = q / (float)cols;
    const float rstd = 1.0f / sqrtf(var + eps);
    for (uint32_t c = 0; c < cols; ++c) {
      const float d = bf16_to_f32(xr[c]) - mean;
      yr[c] = f32_to_bf16(d * rstd * bf16_to_f32(gamma[c]) + bf16_to_f32(beta[c]));
    }
  }
}

ORC_API void orc_layernorm_rows_bf16(const uint16_t* x, const uint16_t* gamma, const uint16_t* beta, uint32_t rows, uint32_t cols, float eps, uint16_t* y) {
  const orc_layernorm_rows_bf16_ctx ctx__ = {x, gamma, beta, rows, cols, eps, y};
  parallel_rows((int64_t)rows, orc_layernorm_rows_bf16_body, &ctx__);
}

/* Same with fp32 rows in and out (the statistics are fp32 either way). */
typedef struct {
  const float* x;
  const float* gamma;
  const float* beta;
  uint32_t rows;
  uint32_t cols;
  float eps;
  float* y;
} orc_layernorm_rows_f32_ctx;

static void orc_layernorm_rows_f32_body(const void* p, int64_t lo, int64_t hi) {
  const orc_layernorm_rows_f32_ctx* q__ = (const orc_layernorm_rows_f32_ctx*)p;
  const float* x = q__->x;
  const float* gamma = q__->gamma;
  const float* beta = q__->beta;
  uint32_t rows = q__->rows;
  uint32_t cols = q__->cols;
  float eps = q__->eps;
  float* y = q__->y;
  (void)x;
  (void)gamma;
  (void)beta;
  (void)rows;
  (void)cols;
  (void)eps;
  (void)y;
  for (int64_t r = lo; r < hi; ++r) {
    const float* xr = x + (size_t)r * cols;
    float* yr = y + (size_t)r * cols;
    float s = 0.0f;
    for (uint32_t c = 0; c < cols; ++c) s += xr[c];
    const float mean = s / (float)cols;
    float q = 0.0f;
    for (uint32_t c = 0; c < cols; ++c) {
      const float d = xr[c] - mean;
      q += d * d;
    }
    const float var = q / (float)cols;
    const float rstd = 1.0f / sqrtf(var + eps);
    for (uint32_t c = 0; c < cols; ++c) yr[c] = (xr[c] - mean) * rstd * gamma[c] + beta[c];
  }
}

ORC_API void orc_layernorm_rows_f32(const float* x, const float* gamma, const float* beta, uint32_t rows, uint32_t cols, float eps, float* y) {
  const orc_layernorm_rows_f32_ctx ctx__ = {x, gamma, beta, rows, cols, eps, y};
  parallel_rows((int64_t)rows, orc_layernorm_rows_f32_body, &ctx__);
}

/* Outer-axis reduce of t[b, k, c] over k: sum, max and argmax in one pass.
 * Loop shape: testing/runners/softmax.cu:49-61 and row_sum.cu (the reduced
 * axis is the MIDDLE one, parked last by `as`; fp32 acc, k ascending). Argmax
 * keeps the lowest index among equal maxima (strict > on update). Any of the
 * three outputs may be NULL. With k == 0: sum = 0, max = -inf, argmax = 0. */
typedef struct {
  const float* t;
  uint32_t nb;
  uint32_t nk;
  uint32_t nc;
  float* sum;
  float* mx;
  int32_t* amax;
} orc_reduce_outer_ctx;

static void orc_reduce_outer_body(const void* p, int64_t lo, int64_t hi) {
  const orc_reduce_outer_ctx* q__ = (const orc_reduce_outer_ctx*)p;
  const float* t = q__->t;
  uint32_t nb = q__->nb;
  uint32_t nk = q__->nk;
  uint32_t nc = q__->nc;
  float* sum = q__->sum;
  float* mx = q__->mx;
  int32_t* amax = q__->amax;
  (void)t;
  (void)nb;
  (void)nk;
  (void)nc;
  (void)sum;
  (void)mx;
  (void)amax;
  for (int64_t b = lo; b < hi; ++b) {
    for (uint32_t c = 0; c < nc; ++c) {
      float acc = 0.0f;
      float best = -INFINITY;
      int32_t bi = 0;
      for (uint32_t k = 0; k < nk; ++k) {
        const float v = t[((size_t)b * nk + k) * nc + c];
        acc += v;
        if (v > best) {
          best = v;
          bi = (int32_t)k;
        }
      }
      const size_t o = (size_t)b * nc + c;
      if (sum) sum[o] = acc;
      if (mx) mx[o] = best;
      if (amax) amax[o] = bi;
    }
  }
}

ORC_API void orc_reduce_outer(const float* t, uint32_t nb, uint32_t nk, uint32_t nc, float* sum, float* mx, int32_t* amax) {
  const orc_reduce_outer_ctx ctx__ = {t, nb, nk, nc, sum, mx, amax};
  parallel_rows((int64_t)nb, orc_reduce_outer_body, &ctx__);
}

typedef struct {
  const float* t;
  uint32_t nb;
  uint32_t nk;
  uint32_t nc;
  double* sum;
  double* sum_abs;
} orc_reduce_outer_sum_f64_ctx;

static void orc_reduce_outer_sum_f64_body(const void* p, int64_t lo, int64_t hi) {
  const orc_reduce_outer_sum_f64_ctx* q__ = (const orc_reduce_outer_sum_f64_ctx*)p;
  const float* t = q__->t;
  uint32_t nb = q__->nb;
  uint32_t nk = q__->nk;
  uint32_t nc = q__->nc;
  double* sum = q__->sum;
  double* sum_abs = q__->sum_abs;
  (void)t;
  (void)nb;
  (void)nk;
  (void)nc;
  (void)sum;
  (void)sum_abs;
  for (int64_t b = lo; b < hi; ++b) {
    for (uint32_t c = 0; c < nc; ++c) {
      double acc = 0.0, aa = 0.0;
      for (uint32_t k = 0; k < nk; ++k) {
        const double v = (double)t[((size_t)b * nk + k) * nc + c];
        acc += v;
        aa += fabs(v);
      }
      sum[(size_t)b * nc + c] = acc;
      if (sum_abs) sum_abs[(size_t)b * nc + c] = aa;
    }
  }
}

ORC_API void orc_reduce_outer_sum_f64(const float* t, uint32_t nb, uint32_t nk, uint32_t nc, double* sum, double* sum_abs) {
  const orc_reduce_outer_sum_f64_ctx ctx__ = {t, nb, nk, nc, sum, sum_abs};
  parallel_rows((int64_t)nb, orc_reduce_outer_sum_f64_body, &ctx__);
}

/* Contraction with a fused epilogue: c = act(a @ b + bias), bf16 operands
 * widened to fp32, fp32 accumulator, k ascending per output, bf16 result.
 * Loop body: testing/runners/gemm.cu:44-56 and the piped map of
 * internal/e2e/frontend_test.go:194-209. The loops run i-k-j over an fp32
 * scratch row so that the CPU finishes in reasonable time; each output still
 * receives its products in ascending k, so every value equals the i-j-k loop's.
 * a is [m,k], b is [k,n] (both row-major), bias is [n] fp32 or NULL.
 * act: 0 = none, 1 = relu via fmaxf(v, 0). */
typedef struct {
  const uint16_t* a;
  const uint16_t* b;
  const float* bias;
  uint32_t m;
  uint32_t n;
  uint32_t k;
  int act;
  uint16_t* c;
} orc_gemm_bias_act_bf16_ctx;

static void orc_gemm_bias_act_bf16_body(const void* p, int64_t lo, int64_t hi) {
  const orc_gemm_bias_act_bf16_ctx* q__ = (const orc_gemm_bias_act_bf16_ctx*)p;
  const uint16_t* a = q__->a;
  const uint16_t* b = q__->b;
  const float* bias = q__->bias;
  uint32_t m = q__->m;
  uint32_t n = q__->n;
  uint32_t k = q__->k;
  int act = q__->act;
  uint16_t* c = q__->c;
  (void)a;
  (void)b;
  (void)bias;
  (void)m;
  (void)n;
  (void)k;
  (void)act;
  (void)c;
  for (int64_t i = lo; i < hi; ++i) {
    float* acc = (float*)malloc((size_t)n * 2 * sizeof(float));
    float* brow = acc + n;
    {
      for (uint32_t j = 0; j < n; ++j) acc[j] = 0.0f;
      for (uint32_t kk = 0; kk < k; ++kk) {
        const float av = bf16_to_f32(a[(size_t)i * k + kk]);
        const uint16_t* bp = b + (size_t)kk * n;
        for (uint32_t j = 0; j < n; ++j) brow[j] = bf16_to_f32(bp[j]);
        for (uint32_t j = 0; j < n; ++j) acc[j] += av * brow[j];
      }
      for (uint32_t j = 0; j < n; ++j) {
        float v = acc[j] + (bias ? bias[j] : 0.0f);
        if (act == 1) v = fmaxf(v, 0.0f);
        c[(size_t)i * n + j] = f32_to_bf16(v);
      }
    }
    free(acc);
  }
}

ORC_API void orc_gemm_bias_act_bf16(const uint16_t* a, const uint16_t* b, const float* bias, uint32_t m, uint32_t n, uint32_t k, int act, uint16_t* c) {
  const orc_gemm_bias_act_bf16_ctx ctx__ = {a, b, bias, m, n, k, act, c};
  parallel_rows((int64_t)m, orc_gemm_bias_act_bf16_body, &ctx__);
}

/* fp32 matmul with an optional piped scale: out[m,q] = scale * sum_n lhs[m,n]*rhs[n,q]
 * -- internal/e2e/frontend_test.go:194-209, testing/runners/gemm.cu:44-56. */
typedef struct {
  const float* lhs;
  const float* rhs;
  uint32_t m;
  uint32_t n;
  uint32_t q;
  float scale;
  float* out;
} orc_matmul_scale_f32_ctx;

static void orc_matmul_scale_f32_body(const void* p, int64_t lo, int64_t hi) {
  const orc_matmul_scale_f32_ctx* q__ = (const orc_matmul_scale_f32_ctx*)p;
  const float* lhs = q__->lhs;
  const float* rhs = q__->rhs;
  uint32_t m = q__->m;
  uint32_t n = q__->n;
  uint32_t q = q__->q;
  float scale = q__->scale;
  float* out = q__->out;
  (void)lhs;
  (void)rhs;
  (void)m;
  (void)n;
  (void)q;
  (void)scale;
  (void)out;
  for (int64_t mi = lo; mi < hi; ++mi) {
    for (uint32_t qi = 0; qi < q; ++qi) {
      float acc = 0.0f;
      for (uint32_t ni = 0; ni < n; ++ni) acc += lhs[(size_t)mi * n + ni] * rhs[(size_t)ni * q + qi];
      out[(size_t)mi * q + qi] = acc * scale;
    }
  }
}

ORC_API void orc_matmul_scale_f32(const float* lhs, const float* rhs, uint32_t m, uint32_t n, uint32_t q, float scale, float* out) {
  const orc_matmul_scale_f32_ctx ctx__ = {lhs, rhs, m, n, q, scale, out};
  parallel_rows((int64_t)m, orc_matmul_scale_f32_body, &ctx__);
}

/* ------------------------------------------------------------------------ */
/* the reference's 14 suite kernels (testing/suite.toml), inputs given         */
/* ------------------------------------------------------------------------ */

enum {
  ORC_SUITE_DUP_EXPR = 0,   /* testing/runners/dup_expr.cu   */
  ORC_SUITE_DUP_CONST = 1,  /* testing/runners/dup_const.cu  */
  ORC_SUITE_AXPY3 = 2,      /* testing/runners/axpy3.cu      */
  ORC_SUITE_MLP = 3,        /* testing/runners/mlp.cu        */
  ORC_SUITE_SOFTMAX = 4,    /* testing/runners/softmax.cu    */
  ORC_SUITE_MM = 5,         /* mm_small / mm_mid / mm_splitk / gemm .cu */
  ORC_SUITE_TRANSPOSE = 6,  /* testing/runners/transpose.cu  */
  ORC_SUITE_ROW_SUM = 7,    /* testing/runners/row_sum.cu    */
  ORC_SUITE_SCALE_COPY = 8, /* testing/runners/scale_copy.cu */
  ORC_SUITE_QK_SCORE = 9,   /* testing/runners/qk_score.cu   */
  ORC_SUITE_LAYERNORM = 10  /* testing/runners/layernorm.cu  */
};

/* One entry for all suite kernels. x and z are the two input tensors (the
 * matmul family reads them as lhs and rhs), d0/d1/d2 are the three extents in
 * the order the runner declares them, s[] the scalar captures in the runner's
 * order. Returns 0, or -1 for an unknown kernel id.
 *
 *   reduce over the INNERMOST axis, x,z = [d0, d1, K=d2], out [d0, d1]:
 *     dup_expr, dup_const, axpy3, scale_copy, transpose, layernorm
 *   reduce over the MIDDLE axis, x,z = [d0, K=d1, d2], out [d0, d2]:
 *     softmax, row_sum
 *   contractions, out [M, N]:
 *     mm/mlp: lhs [M=d0, K=d1], rhs [K, N=d2];  qk_score: q [H=d0, D=d1], kk [N=d2, D]
 */
ORC_API int orc_suite(int kernel, const float* x, const float* z, uint32_t d0, uint32_t d1,
                      uint32_t d2, const float* s, float* out) {
  switch (kernel) {
    case ORC_SUITE_DUP_EXPR: { /* dup_expr.cu CPU loop */
      const float gain = s[0], bias = s[1];
      const uint32_t n_out = d0 * d1, dk = d2;
      for (uint32_t i = 0; i < n_out; ++i) {
        float acc = 0.0f;
        for (uint32_t k = 0; k < dk; ++k) {
          const float v = x[(size_t)i * dk + k];
          const float w = z[(size_t)i * dk + k];
          acc += ((v * v + v * v) * gain + (v * v + v * v) * bias) * w;
        }
        out[i] = acc;
      }
      return 0;
    }
    case ORC_SUITE_DUP_CONST: { /* dup_const.cu CPU loop */
      const uint32_t n_out = d0 * d1, dk = d2;
      for (uint32_t i = 0; i < n_out; ++i) {
        float acc = 0.0f;
        for (uint32_t k = 0; k < dk; ++k) {
          const float v = x[(size_t)i * dk + k];
          const float w = z[(size_t)i * dk + k];
          acc += (0.5f * (v + 0.5f * v * v) * (1.0f + 0.044715f * v) +
                  tanhf(0.79788456f * (v + 0.044715f * v) + 0.79788456f * 0.5f * v) *
                      (1.0f - 0.5f)) *
                 w;
        }
        out[i] = acc;
      }
      return 0;
    }
    case ORC_SUITE_AXPY3: { /* axpy3.cu CPU loop: map | reduce | map */
      const float alpha = s[0], beta = s[1], gamma = s[2];
      const uint32_t n_out = d0 * d1, dk = d2;
      for (uint32_t i = 0; i < n_out; ++i) {
        float v = 0.0f;
        for (uint32_t k = 0; k < dk; ++k)
          v += alpha * x[(size_t)i * dk + k] + beta * z[(size_t)i * dk + k];
        out[i] = v + gamma * tanhf(v);
      }
      return 0;
    }
    case ORC_SUITE_SCALE_COPY: { /* scale_copy.cu CPU loop */
      const float gain = s[0], bias = s[1];
      const uint32_t n_out = d0 * d1, dk = d2;
      for (uint32_t i = 0; i < n_out; ++i) {
        float acc = 0.0f;
        for (uint32_t k = 0; k < dk; ++k)
          acc += (gain * x[(size_t)i * dk + k] + bias) * z[(size_t)i * dk + k];
        out[i] = acc;
      }
      return 0;
    }
    case ORC_SUITE_TRANSPOSE: { /* transpose.cu CPU loop */
      const uint32_t dk = d2;
      for (uint32_t i = 0; i < d0; ++i)
        for (uint32_t j = 0; j < d1; ++j) {
          float acc = 0.0f;
          for (uint32_t k = 0; k < dk; ++k)
            acc += x[((size_t)i * d1 + j) * dk + k] * z[((size_t)i * d1 + j) * dk + k];
          out[(size_t)i * d1 + j] = acc;
        }
      return 0;
    }
    case ORC_SUITE_LAYERNORM: { /* layernorm.cu:47-58 */
      const float inv_n = s[0], eps = s[1];
      const uint32_t n_out = d0 * d1, dk = d2;
      for (uint32_t i = 0; i < n_out; ++i) {
        float acc = 0.0f;
        for (uint32_t k = 0; k < dk; ++k) {
          const float v = x[(size_t)i * dk + k];
          acc += (v * v) * z[(size_t)i * dk + k];
        }
        out[i] = acc * host_rsqrtf(acc * inv_n + eps);
      }
      return 0;
    }
    case ORC_SUITE_SOFTMAX: { /* softmax.cu:49-61 */
      const uint32_t dk = d1, dc = d2;
      for (uint32_t i = 0; i < d0; ++i)
        for (uint32_t j = 0; j < dc; ++j) {
          float acc = 0.0f;
          for (uint32_t k = 0; k < dk; ++k)
            acc += expf(x[((size_t)i * dk + k) * dc + j]) * z[((size_t)i * dk + k) * dc + j];
          out[(size_t)i * dc + j] = acc;
        }
      return 0;
    }
    case ORC_SUITE_ROW_SUM: { /* row_sum.cu CPU loop */
      const uint32_t dk = d1, dc = d2;
      for (uint32_t i = 0; i < d0; ++i)
        for (uint32_t j = 0; j < dc; ++j) {
          float acc = 0.0f;
          for (uint32_t k = 0; k < dk; ++k)
            acc += x[((size_t)i * dk + k) * dc + j] * z[((size_t)i * dk + k) * dc + j];
          out[(size_t)i * dc + j] = acc;
        }
      return 0;
    }
    case ORC_SUITE_MM: /* gemm.cu:44-56, mm_small.cu, mm_mid.cu, mm_splitk.cu */
    case ORC_SUITE_MLP: { /* mlp.cu CPU loop: matmul then tanh-GELU */
      const uint32_t dm = d0, dk = d1, dn = d2;
      for (uint32_t m = 0; m < dm; ++m)
        for (uint32_t n = 0; n < dn; ++n) {
          float acc = 0.0f;
          for (uint32_t k = 0; k < dk; ++k) acc += x[(size_t)m * dk + k] * z[(size_t)k * dn + n];
          if (kernel == ORC_SUITE_MLP) {
            const float u = acc;
            acc = 0.5f * u * (1.0f + tanhf(0.79788456f * (u + 0.044715f * u * u * u)));
          }
          out[(size_t)m * dn + n] = acc;
        }
      return 0;
    }
    case ORC_SUITE_QK_SCORE: { /* qk_score.cu CPU loop */
      const float scale = s[0];
      const uint32_t dh = d0, dd = d1, dn = d2;
      for (uint32_t h = 0; h < dh; ++h)
        for (uint32_t n = 0; n < dn; ++n) {
          float acc = 0.0f;
          for (uint32_t k = 0; k < dd; ++k) acc += x[(size_t)h * dd + k] * z[(size_t)n * dd + k];
          acc *= scale;
          out[(size_t)h * dn + n] = acc;
        }
      return 0;
    }
    default:
      return -1;
  }
}

/* ------------------------------------------------------------------------ */
/* Parity criteria over whole tensors (the per-element rules of oracle/checks.py, */
/* restated in C so that half a billion elements are checked in seconds).         */
/* counts is [rows][5] uint64: checked, failed, passed-only-through-the-added-    */
/* terms, got != want, want != rounded fp64. Rows are independent.                */
/* ------------------------------------------------------------------------ */
static inline double bf16_ulp_of(double v) {
  /* 2 ** (floor(log2 |v|) - 7): the spacing of bf16 values (8 significant bits) at |v| */
  int e;
  double a = fabs(v);
  if (a < 1e-38) a = 1e-38;
  (void)frexp(a, &e); /* a = m * 2**e, m in [0.5, 1) */
  return ldexp(1.0, e - 8);
}

typedef struct {
  const uint16_t* got;
  const uint16_t* want;
  const uint16_t* x;
  const uint16_t* gamma;
  const uint16_t* beta;
  uint32_t cols;
  double eps;
  uint64_t* counts;
} orc_check_ln_ctx;

static void orc_check_layernorm_bf16_body(const void* p, int64_t lo, int64_t hi) {
  const orc_check_ln_ctx* q = (const orc_check_ln_ctx*)p;
  const uint32_t n = q->cols;
  for (int64_t r = lo; r < hi; ++r) {
    const uint16_t* xr = q->x + (size_t)r * n;
    const uint16_t* gr = q->got + (size_t)r * n;
    const uint16_t* wr = q->want + (size_t)r * n;
    uint64_t* c = q->counts + (size_t)r * 5;
    double s = 0.0;
    for (uint32_t j = 0; j < n; ++j) s += (double)bf16_to_f32(xr[j]);
    const double mean = n ? s / n : 0.0;
    double ss = 0.0;
    for (uint32_t j = 0; j < n; ++j) {
      const double d = (double)bf16_to_f32(xr[j]) - mean;
      ss += d * d;
    }
    const double var = n ? ss / n : 0.0;
    const double std = sqrt(var + q->eps);
    uint64_t failed = 0, via = 0, differ = 0, off = 0;
    for (uint32_t j = 0; j < n; ++j) {
      const double g = (double)bf16_to_f32(q->gamma[j]), b = (double)bf16_to_f32(q->beta[j]);
      const double xhat = ((double)bf16_to_f32(xr[j]) - mean) / std;
      const double y64 = xhat * g + b;
      const uint16_t r64b = f32_to_bf16((float)y64);
      const double r64 = (double)bf16_to_f32(r64b);
      const double got = (double)bf16_to_f32(gr[j]), want = (double)bf16_to_f32(wr[j]);
      const double fp32err = 1e-5 * (fabs(xhat * g) + fabs(b)) + 1e-6 * (fabs(mean) / std + 1.0) * fabs(g);
      const double ulp = bf16_ulp_of(fabs(y64) > fabs(got) ? y64 : got);
      const double d_o = fabs(got - want);
      const double ulp_w = bf16_ulp_of(want);
      const int accepted = (fabs(got - y64) <= 0.5 * ulp + fp32err + 1e-30) && (d_o <= ulp_w + fp32err + fabs(want - r64));
      const int bare = d_o <= ulp_w;
      failed += !accepted;
      via += accepted && !bare;
      differ += gr[j] != wr[j];
      off += wr[j] != r64b;
    }
    c[0] = n; c[1] = failed; c[2] = via; c[3] = differ; c[4] = off;
  }
}

ORC_API void orc_check_layernorm_bf16(const uint16_t* got, const uint16_t* want, const uint16_t* x, const uint16_t* gamma,
                                      const uint16_t* beta, uint32_t rows, uint32_t cols, double eps, uint64_t* counts) {
  const orc_check_ln_ctx ctx = {got, want, x, gamma, beta, cols, eps, counts};
  parallel_rows((int64_t)rows, orc_check_layernorm_bf16_body, &ctx);
}

typedef struct {
  const float* got;
  const float* want;
  const float* x;
  uint32_t cols;
  uint64_t* counts;
} orc_check_sm_ctx;

static void orc_check_softmax_body(const void* p, int64_t lo, int64_t hi) {
  const orc_check_sm_ctx* q = (const orc_check_sm_ctx*)p;
  const uint32_t n = q->cols;
  for (int64_t r = lo; r < hi; ++r) {
    const float* xr = q->x + (size_t)r * n;
    const float* gr = q->got + (size_t)r * n;
    const float* wr = q->want + (size_t)r * n;
    uint64_t* c = q->counts + (size_t)r * 5;
    double m = -INFINITY, s = 0.0;
    for (uint32_t j = 0; j < n; ++j) m = (double)xr[j] > m ? (double)xr[j] : m;
    for (uint32_t j = 0; j < n; ++j) s += exp((double)xr[j] - m);
    uint64_t failed = 0, via = 0;
    for (uint32_t j = 0; j < n; ++j) {
      const double f64 = exp((double)xr[j] - m) / s;
      const double got = (double)gr[j], want = (double)wr[j];
      const double d_o = fabs(got - want);
      const int bare = d_o <= 1e-5 * fabs(want) + 1e-37;
      const int accepted = (fabs(got - f64) <= 1e-5 * fabs(f64) + 1e-37) && (d_o <= 1e-5 * fabs(want) + fabs(want - f64) + 1e-37);
      failed += !accepted;
      via += accepted && !bare;
    }
    c[0] = n; c[1] = failed; c[2] = via; c[3] = 0; c[4] = 0;
  }
}

ORC_API void orc_check_softmax(const float* got, const float* want, const float* x, uint32_t rows, uint32_t cols,
                               uint64_t* counts) {
  const orc_check_sm_ctx ctx = {got, want, x, cols, counts};
  parallel_rows((int64_t)rows, orc_check_softmax_body, &ctx);
}
